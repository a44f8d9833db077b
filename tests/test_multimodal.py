import math

import pytest
import torch
import torch.nn.functional as F

from gllm_b200.models.audio import (AudioConfig, AudioWeights, ConformerEncoder, depthwise_conv1d, log_mel_spectrogram,
                                    mel_filterbank)
from gllm_b200.models.multimodal import MultimodalEncoder, MultimodalSpec, expand_placeholders, splice_embeddings
from gllm_b200.models.vision import VisionConfig, VisionTower, VisionWeights, patchify, siglip_tensors


def test_patchify_equals_strided_conv():
    torch.manual_seed(0)
    img = torch.randn(2, 3, 28, 28)
    w = torch.randn(16, 3, 14, 14)
    want = F.conv2d(img, w, stride=14).flatten(2).transpose(1, 2)
    got = patchify(img, 14) @ w.reshape(16, -1).t()
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)


def test_vision_tower_shapes_and_determinism():
    cfg = VisionConfig(image_size=28, patch_size=7, hidden=32, layers=2, heads=4, mlp=64, out_hidden=48, pool=2)
    tower = VisionTower(cfg, VisionWeights(cfg, seed=1))
    img = torch.randn(2, 3, 28, 28)
    out = tower.forward(img)
    assert out.shape == (2, 4, 48) and torch.isfinite(out).all()
    torch.testing.assert_close(tower.forward(img), out)
    # attention is bidirectional: changing the LAST patch changes the FIRST token's output
    img2 = img.clone(); img2[:, :, 21:, 21:] += 1.0
    assert (tower.forward(img2)[:, 0] - out[:, 0]).abs().max() > 1e-6


def test_siglip_checkpoint_names_map_onto_the_tower():
    """A tower stated in plain torch from Hugging Face SigLIP names (conv patch embedding, separate q/k/v) and the
    framework's tower built from the same dict through ``siglip_tensors`` give the same tokens."""
    torch.manual_seed(3)
    cfg = VisionConfig(image_size=28, patch_size=7, hidden=32, layers=2, heads=4, mlp=64, out_hidden=48, pool=2)
    H, P = cfg.hidden, "vision_model."
    ck = {P + "embeddings.patch_embedding.weight": torch.randn(H, 3, 7, 7) * 0.05,
          P + "embeddings.patch_embedding.bias": torch.randn(H) * 0.05,
          P + "embeddings.position_embedding.weight": torch.randn(cfg.num_patches, H) * 0.05,
          P + "post_layernorm.weight": 1 + 0.1 * torch.randn(H), P + "post_layernorm.bias": 0.1 * torch.randn(H),
          "multi_modal_projector.mm_input_projection_weight": torch.randn(H, cfg.out_hidden) * 0.1}
    for l in range(cfg.layers):
        L = f"{P}encoder.layers.{l}."
        for n in ("layer_norm1", "layer_norm2"):
            ck[L + n + ".weight"], ck[L + n + ".bias"] = 1 + 0.1 * torch.randn(H), 0.1 * torch.randn(H)
        for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
            ck[L + f"self_attn.{n}.weight"], ck[L + f"self_attn.{n}.bias"] = torch.randn(H, H) * 0.1, torch.randn(H) * 0.1
        ck[L + "mlp.fc1.weight"], ck[L + "mlp.fc1.bias"] = torch.randn(cfg.mlp, H) * 0.1, torch.randn(cfg.mlp) * 0.1
        ck[L + "mlp.fc2.weight"], ck[L + "mlp.fc2.bias"] = torch.randn(H, cfg.mlp) * 0.1, torch.randn(H) * 0.1
    img = torch.randn(2, 3, 28, 28)

    x = F.conv2d(img, ck[P + "embeddings.patch_embedding.weight"], ck[P + "embeddings.patch_embedding.bias"], stride=7)
    x = x.flatten(2).transpose(1, 2) + ck[P + "embeddings.position_embedding.weight"]
    B, N, _ = x.shape
    heads = lambda t: t.reshape(B, N, cfg.heads, H // cfg.heads).transpose(1, 2)
    for l in range(cfg.layers):
        L = f"{P}encoder.layers.{l}."
        h = F.layer_norm(x, (H,), ck[L + "layer_norm1.weight"], ck[L + "layer_norm1.bias"], cfg.eps)
        q, k, v = (F.linear(h, ck[L + f"self_attn.{n}_proj.weight"], ck[L + f"self_attn.{n}_proj.bias"]) for n in "qkv")
        a = F.scaled_dot_product_attention(heads(q), heads(k), heads(v)).transpose(1, 2).reshape(B, N, H)
        x = x + F.linear(a, ck[L + "self_attn.out_proj.weight"], ck[L + "self_attn.out_proj.bias"])
        h = F.layer_norm(x, (H,), ck[L + "layer_norm2.weight"], ck[L + "layer_norm2.bias"], cfg.eps)
        h = F.gelu(F.linear(h, ck[L + "mlp.fc1.weight"], ck[L + "mlp.fc1.bias"]), approximate="tanh")
        x = x + F.linear(h, ck[L + "mlp.fc2.weight"], ck[L + "mlp.fc2.bias"])
    x = F.layer_norm(x, (H,), ck[P + "post_layernorm.weight"], ck[P + "post_layernorm.bias"], cfg.eps)
    x = F.avg_pool2d(x.reshape(B, cfg.grid, cfg.grid, H).permute(0, 3, 1, 2), 2).flatten(2).transpose(1, 2)
    want = x @ ck["multi_modal_projector.mm_input_projection_weight"]

    t = siglip_tensors(cfg, ck.__getitem__, ck.__contains__)
    assert t["layers.0.qkv.weight"].shape == (3 * H, H) and t["proj.weight"].shape == (cfg.out_hidden, H)
    got = VisionTower(cfg, VisionWeights(cfg, tensors=t)).forward(img)
    torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)


def test_mel_and_conformer():
    fb = mel_filterbank(20, 400, 16000)
    assert fb.shape == (20, 201) and (fb >= 0).all() and (fb.sum(1) > 0).all()
    sr = 16000
    t = torch.arange(sr) / sr
    wave = torch.sin(2 * math.pi * 1000 * t)[None]
    cfg = AudioConfig(n_mels=20, hidden=32, layers=2, heads=4, conv_kernel=7, out_hidden=24)
    mel = log_mel_spectrogram(wave, cfg)
    assert mel.shape[0] == 1 and mel.shape[2] == 20
    peak = int(mel[0].mean(0).argmax())
    centre = [float((fb[i] * torch.linspace(0, 8000, 201)).sum() / fb[i].sum()) for i in range(20)]
    assert abs(centre[peak] - 1000) < 400                        # energy lands in the band around 1 kHz
    x = torch.randn(2, 9, 6); w = torch.randn(6, 1, 3)
    y = depthwise_conv1d(x, w)
    assert y.shape == x.shape
    torch.testing.assert_close(y[0, 4, 2], (x[0, 3:6, 2] * w[2, 0]).sum())
    enc = ConformerEncoder(cfg, AudioWeights(cfg, seed=2))
    out = enc.forward(wave)
    assert out.shape == (1, mel.shape[1] // 4, 24) and torch.isfinite(out).all()


def test_placeholder_expansion_and_splice():
    spec = MultimodalSpec(image_token_id=900, audio_token_id=901)
    ids, spans = expand_placeholders([1, 900, 2, 901, 3], spec, [4], [2])
    assert ids == [1, 900, 900, 900, 900, 2, 901, 901, 3] and spans == [("image", 0, 1, 4), ("audio", 0, 6, 2)]
    with pytest.raises(ValueError):
        expand_placeholders([1, 2], spec, [4])
    emb = torch.zeros(9, 8)
    out = splice_embeddings(emb, spans, [torch.ones(4, 8)], [torch.full((2, 8), 2.0)])
    assert out[1:5].eq(1).all() and out[6:8].eq(2).all() and out[0].eq(0).all()
    vcfg = VisionConfig(image_size=14, patch_size=7, hidden=16, layers=1, heads=2, mlp=32, out_hidden=8)
    mm = MultimodalEncoder(vision=VisionTower(vcfg, VisionWeights(vcfg)), spec=spec)
    table = torch.randn(1000, 8)
    ids2, x = mm.prepare([5, 900, 6], table, images=torch.randn(1, 3, 14, 14))
    assert len(ids2) == 6 and x.shape == (6, 8) and torch.equal(x[0], table[5]) and not torch.equal(x[1], table[900])


def test_client_generation_with_image_input():
    from gllm_b200.client import Client
    from gllm_b200.engine.simple_generate import generate_single
    from gllm_b200.models.config import preset
    from gllm_b200.models.weights import RandomWeights
    cfg = preset("tiny-llama")
    c = Client.from_model(cfg, RandomWeights(cfg, "cpu", torch.float32, seed=3, std=0.05), device="cpu", dtype=torch.float32,
                          max_num_seqs=2, max_model_len=256, max_batch_tokens=64)
    # plain generation through generate_single equals the engine's greedy output
    ids = c.encode("hello world")
    eng = c.generate("hello world").max_tokens(6).temperature(0.0).generate()
    assert generate_single(c._st().model, ids, 6)[:len(eng.token_ids)] == eng.token_ids
    img_tok = 900
    vcfg = VisionConfig(image_size=14, patch_size=7, hidden=16, layers=1, heads=2, mlp=32, out_hidden=cfg.hidden_size)
    c.set_multimodal_encoder(MultimodalEncoder(vision=VisionTower(vcfg, VisionWeights(vcfg, seed=1)),
                                               spec=MultimodalSpec(image_token_id=img_tok)))
    c._prompt_ids = lambda prompt: [5, img_tok, 6, 7]          # a prompt with one image placeholder
    img_a, img_b = torch.randn(3, 14, 14), torch.randn(3, 14, 14) * 3
    ra = c.generate("x").max_tokens(5).temperature(0.0).image(img_a).generate()
    ra2 = c.generate("x").max_tokens(5).temperature(0.0).image(img_a).generate()
    rb = c.generate("x").max_tokens(5).temperature(0.0).image(img_b).generate()
    assert ra.prompt_tokens == 3 + 4 and ra.token_ids == ra2.token_ids and len(ra.token_ids) >= 1
    assert len(rb.token_ids) >= 1
    with pytest.raises(Exception):
        Client.from_model(cfg, RandomWeights(cfg, "cpu", torch.float32, seed=3), device="cpu", dtype=torch.float32,
                          max_num_seqs=2, max_model_len=64, max_batch_tokens=32).generate("x").image(img_a).max_tokens(2).generate()


def test_client_builds_the_image_encoder_from_a_multimodal_checkpoint(tmp_path):
    """A directory with a llava / gemma3 style layout (language model under ``language_model.``, SigLIP tower under
    ``vision_tower.vision_model.``, projector beside them, ``vision_config`` in config.json): the client loads the
    decoder AND attaches the image encoder, and a prompt with the image placeholder generates."""
    import json
    from gllm_b200.client import Client
    from gllm_b200.loader import safetensors as st
    from gllm_b200.models.config import preset
    from tests.test_loaders import _hf_state
    cfg = preset("tiny-qwen3")
    _, sd = _hf_state(cfg)
    sd = {"language_model." + k: v for k, v in sd.items()}
    g = torch.Generator().manual_seed(5)
    r = lambda *s: torch.randn(*s, generator=g) * 0.05
    Hv, P = 16, "vision_tower.vision_model."
    sd.update({P + "embeddings.patch_embedding.weight": r(Hv, 3, 7, 7), P + "embeddings.patch_embedding.bias": r(Hv),
               P + "embeddings.position_embedding.weight": r(4, Hv), P + "post_layernorm.weight": torch.ones(Hv),
               P + "post_layernorm.bias": torch.zeros(Hv), "multi_modal_projector.linear.weight": r(cfg.hidden_size, Hv)})
    L = P + "encoder.layers.0."
    for n in ("layer_norm1", "layer_norm2"):
        sd[L + n + ".weight"], sd[L + n + ".bias"] = torch.ones(Hv), torch.zeros(Hv)
    for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
        sd[L + f"self_attn.{n}.weight"], sd[L + f"self_attn.{n}.bias"] = r(Hv, Hv), r(Hv)
    sd[L + "mlp.fc1.weight"], sd[L + "mlp.fc1.bias"], sd[L + "mlp.fc2.weight"], sd[L + "mlp.fc2.bias"] = r(32, Hv), r(32), r(Hv, 32), r(Hv)
    d = tmp_path / "mm"
    d.mkdir()
    st.save_file(sd, d / "model.safetensors")
    (d / "config.json").write_text(json.dumps({
        "model_type": "llava", "image_token_index": 900,
        "text_config": {"model_type": "qwen3", "hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 4,
                        "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 512, "vocab_size": 1024,
                        "rope_theta": 1e6, "rms_norm_eps": 1e-6, "max_position_embeddings": 2048, "eos_token_id": 2,
                        "tie_word_embeddings": False},
        "vision_config": {"image_size": 14, "patch_size": 7, "hidden_size": Hv, "num_hidden_layers": 1,
                          "num_attention_heads": 2, "intermediate_size": 32}}))
    c = Client.builder().model(str(d)).backend("cpu").config(max_num_seqs=2, max_model_len=128, max_batch_tokens=64).build()
    enc = c._multimodal_encoder
    assert enc is not None and enc.spec.image_token_id == 900 and enc.vision.cfg.out_hidden == cfg.hidden_size
    feats = enc.encode_images(torch.randn(1, 3, 14, 14))
    assert feats[0].shape == (4, cfg.hidden_size)
    c._prompt_ids = lambda prompt: [5, 900, 6]
    out = c.generate("x").max_tokens(3).temperature(0.0).image(torch.randn(3, 14, 14)).generate()
    assert out.prompt_tokens == 2 + 4 and len(out.token_ids) >= 1
