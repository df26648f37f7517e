"""Qwen2-VL vision pipeline (reference: src/models/qwen_vl_vision.cpp, qwen_vl_model.cpp, qwen2_5_vl_image_processor.cpp,
position_inputs.cpp).  The oracle is the checkpoint family's own implementation in `transformers`, built with a small random
configuration: same weights, same patches, same grids."""
import numpy as np
import pytest
import torch

from onnxruntime_genai_b200.models import qwen_vl
from onnxruntime_genai_b200.models.qwen_vl import QwenVisionConfig, QwenVisionTower

hf_modeling = pytest.importorskip("transformers.models.qwen2_vl.modeling_qwen2_vl")
hf_config = pytest.importorskip("transformers.models.qwen2_vl.configuration_qwen2_vl")

CFG = QwenVisionConfig(depth=2, embed_dim=32, hidden_size=48, num_heads=4, mlp_ratio=2.0, patch_size=14, spatial_merge_size=2,
                       temporal_patch_size=2, min_pixels=28 * 28, max_pixels=28 * 28 * 16)


def _hf_tower():
    c = hf_config.Qwen2VLVisionConfig(depth=CFG.depth, embed_dim=CFG.embed_dim, hidden_size=CFG.hidden_size, num_heads=CFG.num_heads,
                                      mlp_ratio=int(CFG.mlp_ratio), in_channels=3, patch_size=14, spatial_merge_size=2, temporal_patch_size=2)
    torch.manual_seed(0)
    m = hf_modeling.Qwen2VisionTransformerPretrainedModel(c).eval()
    with torch.no_grad():
        for p in m.parameters():
            p.copy_(torch.randn_like(p) * 0.1)
    return m


def test_vision_tower_matches_the_checkpoint_familys_implementation(tmp_path):
    hf = _hf_tower()
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    assert set(sd) == set(qwen_vl.weight_shapes(CFG))
    grids = [(1, 4, 6), (1, 2, 2), (2, 2, 4)]
    n = sum(t * h * w for t, h, w in grids)
    patches = torch.randn(n, CFG.patch_dim, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(patches, torch.tensor(grids))
    want = want if isinstance(want, torch.Tensor) else want.pooler_output      # the merged patches
    tower = QwenVisionTower(CFG, sd, "cpu", torch.float32)
    got = tower.forward(patches, grids)
    assert got.shape == (n // 4, CFG.hidden_size)
    torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)
    # through the file format
    path = qwen_vl.export_qwen_vision(CFG, str(tmp_path), sd, precision="fp32")
    assert QwenVisionTower.is_file(path)
    again = QwenVisionTower.load(path, "cpu", torch.float32)
    assert asdict_equal(again.cfg, CFG)
    torch.testing.assert_close(again.forward(patches, grids), got, rtol=1e-5, atol=1e-5)


def test_windowed_vision_tower_matches_the_qwen2_5_vl_implementation():
    """Qwen2.5-VL: RMS norms, gated SiLU MLP, attention inside windows except in the listed blocks; grids whose sides are and are
    not multiples of the window."""
    m25 = pytest.importorskip("transformers.models.qwen2_5_vl.modeling_qwen2_5_vl")
    c25 = pytest.importorskip("transformers.models.qwen2_5_vl.configuration_qwen2_5_vl")
    hc = c25.Qwen2_5_VLVisionConfig(depth=3, hidden_size=32, intermediate_size=48, num_heads=4, in_channels=3, out_hidden_size=40,
                                    patch_size=14, spatial_merge_size=2, temporal_patch_size=2, window_size=56, fullatt_block_indexes=[1],
                                    hidden_act="silu")
    torch.manual_seed(2)
    hf = m25.Qwen2_5_VisionTransformerPretrainedModel(hc).eval()
    with torch.no_grad():
        for p in hf.parameters():
            p.copy_(torch.randn_like(p) * 0.1)
    cfg = QwenVisionConfig(depth=3, embed_dim=32, hidden_size=40, num_heads=4, variant="qwen2_5_vl", intermediate_size=48, window_size=56,
                           fullatt_blocks="1")
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    assert set(sd) == set(qwen_vl.weight_shapes(cfg))
    tower = QwenVisionTower(cfg, sd, "cpu", torch.float32)
    for grids in ([(1, 4, 6), (1, 2, 4)], [(1, 8, 8)], [(2, 6, 10), (1, 2, 2)]):
        n = sum(t * h * w for t, h, w in grids)
        patches = torch.randn(n, cfg.patch_dim, generator=torch.Generator().manual_seed(n))
        with torch.no_grad():
            want = hf(patches, torch.tensor(grids)).pooler_output
        torch.testing.assert_close(tower.forward(patches, grids), want, rtol=3e-4, atol=3e-4)


def asdict_equal(a, b):
    from dataclasses import asdict
    da, db = asdict(a), asdict(b)
    return set(da) == set(db) and all(da[k] == db[k] if isinstance(da[k], str) else abs(da[k] - db[k]) <= 1e-6 * max(1.0, abs(db[k]))
                                      for k in da)   # numeric attributes are stored as fp32


def test_smart_resize_and_patch_layout_match_the_checkpoint_familys_processor():
    hf_ip = pytest.importorskip("transformers.models.qwen2_vl.image_processing_qwen2_vl")
    for h, w in [(56, 56), (300, 500), (31, 640), (1000, 37), (224, 224), (1080, 1920)]:
        assert qwen_vl.smart_resize(h, w, 28, CFG.min_pixels, CFG.max_pixels) == hf_ip.smart_resize(h, w, 28, CFG.min_pixels, CFG.max_pixels)
    # an image already at a valid size goes through normalisation and the patch layout only
    rng = np.random.RandomState(0)
    img = rng.randint(0, 256, size=(56, 84, 3), dtype=np.uint8)
    patches, grid = qwen_vl.preprocess_image(img, CFG)
    assert grid == (1, 4, 6) and patches.shape == (24, CFG.patch_dim)
    proc = hf_ip.Qwen2VLImageProcessor(min_pixels=CFG.min_pixels, max_pixels=CFG.max_pixels, patch_size=14, merge_size=2, temporal_patch_size=2)
    out = proc(images=[img], return_tensors="pt")
    assert out["image_grid_thw"].tolist() == [[1, 4, 6]]
    torch.testing.assert_close(patches, out["pixel_values"].float(), rtol=1e-5, atol=1e-5)
    # a resized image: same grid, pixels close (the two bicubic filters differ slightly)
    img2 = rng.randint(0, 256, size=(100, 150, 3), dtype=np.uint8)
    p2, g2 = qwen_vl.preprocess_image(img2, CFG)
    o2 = proc(images=[img2], return_tensors="pt")
    assert [list(g2)] == o2["image_grid_thw"].tolist() and p2.shape == o2["pixel_values"].shape
    assert (p2 - o2["pixel_values"].float()).abs().mean() < 0.08


def test_mrope_positions_follow_the_checkpoint_familys_rule():
    """Text advances all three components; an image keeps the temporal one, takes row / column of the merged patch, and the text
    after it continues one past the largest component.  Checked against transformers' get_rope_index on a prompt with two images."""
    IMG, START, END = 90, 91, 92
    grids = [(1, 4, 6), (1, 2, 4)]
    toks = [5, 6, START] + [IMG] * 6 + [END, 7, 8, START] + [IMG] * 2 + [END, 9]
    pos, used, nxt = qwen_vl.mrope_positions(toks, IMG, grids, 2)
    assert used == 2
    cfg = hf_config.Qwen2VLConfig(vocab_size=100, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
                                  num_key_value_heads=2, image_token_id=IMG, video_token_id=93, vision_start_token_id=START,
                                  vision_end_token_id=END,
                                  vision_config=dict(depth=1, embed_dim=32, hidden_size=32, num_heads=4, mlp_ratio=2, patch_size=14,
                                                     spatial_merge_size=2, temporal_patch_size=2),
                                  rope_scaling={"type": "mrope", "mrope_section": [2, 1, 1]})
    model = hf_modeling.Qwen2VLModel(cfg)
    ids = torch.tensor([toks])
    types = (ids == IMG).int()                          # text 0, image 1
    want, delta = model.get_rope_index(ids, mm_token_type_ids=types, image_grid_thw=torch.tensor(grids), attention_mask=torch.ones_like(ids))
    assert pos.tolist() == want[:, 0, :].tolist()
    assert nxt - len(toks) == int(delta.reshape(-1)[0])
    with pytest.raises(RuntimeError):
        qwen_vl.mrope_positions([IMG] * 5, IMG, [(1, 4, 6)], 2)


def test_generator_with_an_image_follows_the_dense_reference(tmp_path):
    """End to end on the CPU: patches + grid + prompt through `Generator.set_inputs`.  The oracle assembles the same step by
    hand - the checkpoint family's own vision tower for the features, its own position rule, the dense decoder reference with the
    image rows of the embedding replaced - and the generated tokens continue one past the largest position component."""
    import copy
    import sys
    sys.path.insert(0, __import__("os").path.dirname(__file__))
    from dense_reference import logits as dense_logits
    import onnxruntime_genai_b200 as og
    from onnxruntime_genai_b200.models.arch import ArchConfig
    from onnxruntime_genai_b200.models.builder import export_qwen_vl, random_state_dict
    IMG = 200
    arch = ArchConfig(model_type="qwen2_vl", vocab_size=211, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
                      intermediate_size=128, context_length=256, bos_token_id=0, eos_token_id=210, pad_token_id=0, attn_bias=True,
                      mrope_section=[2, 3, 3])
    vis = QwenVisionConfig(depth=2, embed_dim=32, hidden_size=64, num_heads=4, mlp_ratio=2.0, min_pixels=28 * 28, max_pixels=28 * 28 * 16)
    hf_cfg = hf_config.Qwen2VLVisionConfig(depth=2, embed_dim=32, hidden_size=64, num_heads=4, mlp_ratio=2, in_channels=3, patch_size=14,
                                           spatial_merge_size=2, temporal_patch_size=2)
    torch.manual_seed(3)
    hf = hf_modeling.Qwen2VisionTransformerPretrainedModel(hf_cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():
            p.copy_(torch.randn_like(p) * 0.1)
    vsd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    sd = random_state_dict(arch, seed=13, std=0.15)
    d = str(tmp_path)
    export_qwen_vl(copy.deepcopy(arch), vis, d, IMG, "fp32", "cpu", decoder_state_dict=sd, vision_state_dict=vsd)
    model = og.Model(d)
    assert model.vision is not None and model.image_token_id == IMG

    rng = np.random.RandomState(4)
    img_a, img_b = rng.randint(0, 256, size=(56, 84, 3), dtype=np.uint8), rng.randint(0, 256, size=(28, 56, 3), dtype=np.uint8)
    (pa, ga), (pb, gb) = qwen_vl.preprocess_image(img_a, vis), qwen_vl.preprocess_image(img_b, vis)
    assert ga == (1, 4, 6) and gb == (1, 2, 4)
    ids = [5, 6] + [IMG] * 6 + [7, 8, 9] + [IMG] * 2 + [11]
    patches, grids = torch.cat([pa, pb]), [ga, gb]

    p = og.GeneratorParams(model)
    p.set_search_options(max_length=40)
    g = og.Generator(model, p)
    g.set_inputs({"pixel_values": patches.numpy(), "image_grid_thw": np.asarray(grids, dtype=np.int64),
                  "input_ids": np.asarray([ids], dtype=np.int32)})

    with torch.no_grad():
        feats = hf(patches, torch.tensor(grids)).pooler_output
    emb = sd["model.embed_tokens.weight"].float()[torch.tensor(ids)].clone()
    emb[torch.tensor(ids) == IMG] = feats
    p3, used, nxt = qwen_vl.mrope_positions(ids, IMG, grids, 2)
    want = dense_logits(arch, sd, ids, inputs_embeds=emb, positions3=p3)[-1].numpy()
    np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=2e-3, atol=5e-4)
    assert g.state.rope_delta[0] == nxt - len(ids)
    g.generate_next_token()
    tok = int(g.get_next_tokens()[0])
    emb2 = torch.cat([emb, sd["model.embed_tokens.weight"].float()[tok][None]])
    p3b = np.concatenate([p3, np.full((3, 1), nxt, dtype=np.int32)], axis=1)
    want = dense_logits(arch, sd, ids + [tok], inputs_embeds=emb2, positions3=p3b)[-1].numpy()
    np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=2e-3, atol=6e-4)
    # fewer image tokens than the grids say is refused
    g2 = og.Generator(model, p)
    with pytest.raises(RuntimeError):
        g2.set_inputs({"pixel_values": pa.numpy(), "image_grid_thw": np.asarray([ga], dtype=np.int64),
                       "input_ids": np.asarray([[5] + [IMG] * 4 + [7]], dtype=np.int32)})


def test_hf_checkpoint_directory_exports_decoder_and_tower(tmp_path):
    """A Qwen2.5-VL checkpoint directory (config.json with text_config / vision_config, `model.language_model.*` and `model.visual.*`
    tensors) through create_model: the decoder and the vision tower are exported together, and a prompt with an image gives the logits
    of the family's own implementation (patch features spliced into the prompt, three-component rotary positions)."""
    import json
    from safetensors.torch import save_file
    transformers = pytest.importorskip("transformers")
    if not hasattr(transformers, "Qwen2_5_VLForConditionalGeneration"):
        pytest.skip("transformers has no Qwen2_5_VLForConditionalGeneration")
    import onnxruntime_genai_b200 as og
    from onnxruntime_genai_b200.models.builder import create_model
    IMG = 110
    cfg = transformers.Qwen2_5_VLConfig(
        text_config=dict(vocab_size=120, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         max_position_embeddings=256, rope_parameters={"rope_type": "default", "mrope_section": [2, 3, 3], "rope_theta": 10000.0},
                         tie_word_embeddings=False, bos_token_id=0, eos_token_id=119, pad_token_id=0),
        vision_config=dict(depth=2, hidden_size=32, out_hidden_size=64, num_heads=2, intermediate_size=48, patch_size=14, spatial_merge_size=2,
                           temporal_patch_size=2, window_size=56, fullatt_block_indexes=[1], in_channels=3, tokens_per_second=1),
        image_token_id=IMG, video_token_id=111, vision_start_token_id=108, vision_end_token_id=109, tie_word_embeddings=False)
    # (tokens_per_second = 1: a still image's temporal position is the position where the image starts, as in the family's published
    # position rule and the reference's src/models/position_inputs.cpp; some transformers versions scale that start by the rate)
    torch.manual_seed(0)
    m = transformers.Qwen2_5_VLForConditionalGeneration(cfg).float().eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            p.copy_(1 + 0.1 * torch.randn_like(p) if ("norm" in n and n.endswith("weight")) else torch.randn_like(p) * 0.1)
    src = tmp_path / "hf"
    src.mkdir()
    save_file({k: v.detach().clone().contiguous() for k, v in m.state_dict().items()}, str(src / "model.safetensors"))
    d = cfg.to_dict()
    d["architectures"] = ["Qwen2_5_VLForConditionalGeneration"]
    (src / "config.json").write_text(json.dumps(d))
    out = str(tmp_path / "out")
    create_model(str(src), out, "fp32", "cpu")
    model = og.Model(out)
    assert model.type == "qwen2_5_vl" and model.vision is not None and model.image_token_id == IMG and model.arch.mrope_section == [2, 3, 3]

    vis = model.vision.cfg
    rng = np.random.RandomState(4)
    patches, grid = qwen_vl.preprocess_image(rng.randint(0, 256, size=(56, 84, 3), dtype=np.uint8), vis)
    assert grid == (1, 4, 6)
    ids = [5, 108] + [IMG] * 6 + [109, 7, 8, 9]
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=32)
    g = og.Generator(model, p)
    g.set_inputs({"pixel_values": patches.numpy(), "image_grid_thw": np.asarray([grid], dtype=np.int64), "input_ids": np.asarray([ids], dtype=np.int32)})
    with torch.no_grad():
        kw = dict(input_ids=torch.tensor([ids]), pixel_values=patches, image_grid_thw=torch.tensor([grid]))
        try:
            want = m(**kw, mm_token_type_ids=torch.tensor([[1 if t == IMG else 0 for t in ids]])).logits[0, -1].float().numpy()
        except TypeError:
            want = m(**kw).logits[0, -1].float().numpy()
    np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=3e-3, atol=5e-4)
