"""Model directories without a GPU: the safetensors container, the configuration reader, the architecture registry,
the random-model writer, and the oracle's own consistency."""
import json
import math
import os

import pytest
import torch

import layered_oracle as O
from dllama_b200.formats.safetensors import SafetensorsFile, write_safetensors
from dllama_b200.models import registry
from dllama_b200.models.layered import LayerListConfig, example_config, random_tensors, write_random_model


def test_safetensors_round_trip(tmp_path):
    t = {"a.b": torch.randn(3, 5).to(torch.bfloat16), "c": torch.arange(7, dtype=torch.int32), "d": torch.randn(2, 2, 2),
         "e": torch.randn(4).to(torch.float16)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t)
    with open(p, "rb") as f:
        n = int.from_bytes(f.read(8), "little")
        head = json.loads(f.read(n))
    assert head["a.b"] == {"dtype": "BF16", "shape": [3, 5], "data_offsets": head["a.b"]["data_offsets"]}
    st = SafetensorsFile(p)
    assert set(st.names()) == set(t) and st.shape("d") == (2, 2, 2) and "zz" not in st
    for k, v in t.items():
        assert st.tensor(k).dtype == v.dtype and torch.equal(st.tensor(k), v)
    st.close()
    with open(p, "r+b") as f:                       # a tensor whose byte range does not match its shape is refused
        f.seek(8)
        f.write(json.dumps(head).replace('"shape":[3,5]', '"shape":[3,6]').encode()[:n])
    with pytest.raises(ValueError):
        SafetensorsFile(p).tensor("a.b")


def test_configuration_and_registry(tmp_path):
    cfg = example_config(blocks=3)
    d = str(tmp_path / "m")
    tensors = write_random_model(d, cfg, seed=1)
    assert registry.is_model_dir(d) and not registry.is_model_dir(str(tmp_path / "nope"))
    assert registry.architecture_of(d) == "Ribivik" and "Ribivik" in registry.ARCHITECTURES
    c = LayerListConfig.load(d)
    assert c.vocab_size == cfg["vocab"] and c.n_layers == 6 and c.layers[1].mlp is None and c.layers[4].mixer["kv_from"] == 0
    assert "l4.mix.dkv" not in tensors and "l0.mix.dkv" in tensors and "l1.mlp.up" not in tensors and "l3.mlp.up" in tensors
    assert tensors["l1.mix.in"].shape == (2 * 96 + 2 * 2 * 16 + 4, 192) and tensors["l0.mix.uq"].shape == (4 * 48, 48)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump({**cfg, "architecture": "NoSuchDesign"}, f)
    with pytest.raises(ValueError):
        registry.engine_for_dir(d)


def test_oracle_prefix_property():
    """Causality of the oracle itself: the logits of a prefix do not change when tokens are appended."""
    cfg = example_config(width=48, vocab=40, blocks=3, heads=2)
    t = random_tensors(cfg, seed=2)
    toks = torch.randint(0, 40, (20,), generator=torch.Generator().manual_seed(3)).tolist()
    a, b = O.model_logits(t, cfg, toks), O.model_logits(t, cfg, toks[:11])
    assert torch.allclose(a[:11], b, atol=1e-9)


# ---- Sunesun: configuration, weight names, frequency table, the oracle's own window --------------------------------------
def test_sunesun_configuration_weights_of_and_streams(tmp_path):
    import sunesun_oracle as S
    from dllama_b200.models.layered import example_config_sunesun, interpolated_rotary
    cfg = example_config_sunesun(layers=3, streams=2)
    d = str(tmp_path / "s")
    tensors = write_random_model(d, cfg, seed=1)
    assert registry.architecture_of(d) == "Sunesun" and "Sunesun" in registry.ARCHITECTURES
    c = LayerListConfig.load(d)
    assert (c.residual, c.streams, c.hyper_weights, c.embed_scale, c.residual_mult) == ("hyper", 2, True, 2.0, 0.5)
    assert [l.weights_of for l in c.layers] == [None, None, 0]
    assert "l2.mix.q" not in tensors and "l2.hc1.mix" not in tensors and tensors["l1.hc2.mix"].shape == (2, 2)
    assert tensors["l0.mix.k"].shape == (3 * 32, 160) and tensors["l0.mlp.e11.down"].shape == (160, 64) and "l0.mix.v" not in tensors
    plain = {k: v for k, v in cfg.items() if k != "streams"}
    c2 = LayerListConfig.from_dict(plain)
    assert c2.streams == 1 and not c2.hyper_weights and "l0.hc1.in" not in random_tensors(plain, seed=1)
    bad = json.loads(json.dumps(cfg))
    bad["layers"][1]["weights_of"] = 2                      # a layer that has no weights of its own
    with pytest.raises(ValueError):
        LayerListConfig.from_dict(bad)
    # the engine's frequency table equals the oracle's angles
    rot = cfg["layers"][0]["mixer"]["rot"]
    f, mag = interpolated_rotary(rot["base"], rot["dims"], rot["scaling"])
    cos, sin = S.rotary_table(rot, 50)
    pos = torch.arange(50, dtype=torch.float64)[:, None]
    assert torch.allclose(torch.cos(pos * f) * mag, cos, atol=1e-12) and torch.allclose(torch.sin(pos * f) * mag, sin, atol=1e-12)
    assert mag > 1.0 and float(f[-1]) < rot["base"] ** (-2.0 * (rot["dims"] // 2 - 1) / rot["dims"])      # slow frequencies were divided


def test_sunesun_oracle_window_and_prefix_property():
    """The oracle itself: appended tokens change nothing before them, and a token outside every window changes nothing."""
    import sunesun_oracle as S
    from dllama_b200.models.layered import example_config_sunesun
    cfg = example_config_sunesun(width=48, vocab=40, layers=2, heads=2, kv_heads=1, window=6, streams=3)
    t = random_tensors(cfg, seed=2)
    toks = torch.randint(0, 40, (30,), generator=torch.Generator().manual_seed(3)).tolist()
    a, b = S.model_logits(t, cfg, toks), S.model_logits(t, cfg, toks[:11])
    assert torch.allclose(a[:11], b, atol=1e-9)
    other = list(toks)
    other[3] = (toks[3] + 1) % 40
    c = S.model_logits(t, cfg, other)
    # two layers of window 6 reach 10 positions back: position 3 is seen up to position 13 and by nothing after it
    assert not torch.allclose(a[13], c[13], atol=1e-9) and torch.allclose(a[14:], c[14:], atol=1e-9)


# ---- Venadra: configuration, design traits, weight names, the oracle's own chunks and recurrence ----------------------------
def test_venadra_configuration_traits_and_tensor_names(tmp_path):
    from dllama_b200.models.layered import DESIGNS, example_config_venadra
    cfg = example_config_venadra()
    d = str(tmp_path / "v")
    tensors = write_random_model(d, cfg, seed=1)
    assert registry.architecture_of(d) == "Venadra" and "Venadra" in registry.ARCHITECTURES
    c = LayerListConfig.load(d)
    assert (c.residual, c.streams, c.hyper_weights, c.canon_taps, c.embed_scale) == ("hyper", 1, False, 3, 4.0)
    assert c.traits is DESIGNS["Venadra"] and c.traits["attention"]["mask"] == "chunk" and c.traits["moe"]["score"] == "softmax"
    assert [l.weights_of for l in c.layers] == [None, None, None, 0, 1]
    assert tensors["l0.norm1"].dim() == 0 and tensors["final.norm"].dim() == 0 and tensors["l0.canon1"].shape == (160, 3)
    assert tensors["l0.mix.norm"].shape == (3 * 24,) and tensors["l0.mlp.act"].shape == (4,) and tensors["l1.mix.sink"].shape == (6,)
    assert tensors["l1.mix.v"].shape == (3 * 32, 160) and tensors["l1.mlp.e5.gate"].shape == (48, 160)
    assert "l3.mix.q" not in tensors and "l4.canon1" not in tensors and "l0.hc1.in" not in tensors
    # the same mixer types under another design keep that design's meaning: no sink, gate or value projection for Sunesun
    from dllama_b200.models.layered import example_config_sunesun
    assert "l0.mix.sink" not in random_tensors(example_config_sunesun(), seed=1)
    bad = json.loads(json.dumps(cfg))
    bad["layers"][3]["weights_of"] = 4                      # a layer that has no weights of its own
    with pytest.raises(ValueError):
        LayerListConfig.from_dict(bad)


def test_venadra_oracle_chunks_recurrence_and_prefix_property():
    """The oracle itself: appended tokens change nothing before them; through chunked attention and the short convolution
    alone a changed token reaches one chunk further per layer and no more; a lightning layer carries it to the end; the
    recurrence equals its unrolled sum."""
    import venadra_oracle as V
    attn = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 12, "scale": 0.3, "mask": {"size": 6}}
    cfg = {"architecture": "Venadra", "width": 48, "vocab": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0}, "canon": {"taps": 2},
           "layers": [{"type": "attention", "mixer": attn, "mlp": {"kind": "dense", "ff": 32}},
                      {"type": "attention", "mixer": attn, "mlp": None, "weights_of": 0}]}
    cfg["layers"][1]["mlp"] = cfg["layers"][0]["mlp"]
    t = random_tensors(cfg, seed=2)
    toks = torch.randint(0, 40, (30,), generator=torch.Generator().manual_seed(3)).tolist()
    a, b = V.model_logits(t, cfg, toks), V.model_logits(t, cfg, toks[:11])
    assert torch.allclose(a[:11], b, atol=1e-9)
    other = list(toks)
    other[3] = (toks[3] + 1) % 40
    c = V.model_logits(t, cfg, other)
    # layer 0: positions 3..5 (its chunk) and, by the convolution of layer 1, position 6, which layer 1 spreads over chunk 6..11
    assert torch.allclose(a[:3], c[:3], atol=1e-9) and not torch.allclose(a[11], c[11], atol=1e-9) and torch.allclose(a[12:], c[12:], atol=1e-9)
    cfg["layers"][1] = {"type": "lightning", "mixer": {"heads": 2, "dim": 4, "vdim": 6, "decay": [0.99, 0.5]}, "mlp": None}
    t = random_tensors(cfg, seed=2)
    assert not torch.allclose(V.model_logits(t, cfg, toks)[-1], V.model_logits(t, cfg, other)[-1], atol=1e-9)
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(9, n, generator=g, dtype=torch.float64) for n in (4, 4, 6))
    o = V.decayed_linear_attention(q, k, v, 0.8)
    want = sum(0.8 ** (8 - j) * float(q[8] @ k[j]) * v[j] for j in range(9))
    assert torch.allclose(o[8], want, atol=1e-12)


# ---- Darusun: configuration, design traits, weight names, the oracle's own window, head mix and routing -----------------------
def test_darusun_configuration_traits_and_tensor_names(tmp_path):
    from dllama_b200.models.layered import DESIGNS, example_config_darusun
    cfg = example_config_darusun()
    d = str(tmp_path / "d")
    tensors = write_random_model(d, cfg, seed=1)
    assert registry.architecture_of(d) == "Darusun" and "Darusun" in registry.ARCHITECTURES
    c = LayerListConfig.load(d)
    assert (c.residual, c.streams, c.residual_mult, c.canon_taps, c.embed_scale, c.logit_softcap) == ("post", 1, 0.6, 0, 1.0, 0.0)
    assert c.traits is DESIGNS["Darusun"] and c.traits["attention"]["talk"] and c.traits["latent"]["gate"] == "head"
    assert tensors["l0.norm1"].dim() == 0 and tensors["final.norm"].dim() == 0 and "l0.norm1b" not in tensors
    assert tensors["l0.mix.talk"].shape == (6, 6) and tensors["l0.mix.v"].shape == (3 * 48, 160) and tensors["l0.mlp.act"].shape == (2,)
    assert tensors["l1.mix.g"].shape == (4, 160) and tensors["l1.mix.sink"].shape == (4,) and tensors["l1.mix.dkv"].shape == (48 + 8, 160)
    assert tensors["l1.mlp.router.b"].shape == (6,) and tensors["l1.mlp.shared.sg"].shape == (1, 160) and tensors["l1.mlp.e5.gate"].shape == (48, 160)
    assert "l2.mix.k" not in tensors and "l2.mix.v" not in tensors and tensors["l2.mix.q"].shape == (6 * 32, 160)
    # the same mixer types under another design keep that design's meaning: Ribivik's latent attention gates every column
    assert random_tensors(example_config(blocks=1), seed=1)["l0.mix.g"].shape[0] == 4 * 24


def test_darusun_oracle_window_head_mix_routing_and_prefix_property():
    """The oracle itself: appended tokens change nothing before them; through windowed latent layers alone a changed token
    reaches one window further per layer and no more; an identity head mix leaves plain attention; the folded form of the
    mix equals the mix of the scores; the chosen experts' weights sum to one."""
    import darusun_oracle as D
    lat = {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 6, "q_rank": 10, "kv_rank": 12, "scale": 0.3, "rot": {"base": 100.0, "dims": 4}, "mask": {"size": 5}}
    cfg = {"architecture": "Darusun", "width": 48, "vocab": 40, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
           "layers": [{"type": "latent_attention", "mixer": lat, "mlp": {"kind": "dense", "ff": 32}},
                      {"type": "latent_attention", "mixer": lat, "mlp": {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 4, "top": 2}, "shared": {"ff": 12}}}]}
    t = random_tensors(cfg, seed=2)
    toks = torch.randint(0, 40, (30,), generator=torch.Generator().manual_seed(3)).tolist()
    a, b = D.model_logits(t, cfg, toks), D.model_logits(t, cfg, toks[:11])
    assert torch.allclose(a[:11], b, atol=1e-9)
    other = list(toks)
    other[3] = (toks[3] + 1) % 40
    c = D.model_logits(t, cfg, other)
    # layer 0 carries position 3 to 3..7, layer 1 from there to 11 at most
    assert torch.allclose(a[:3], c[:3], atol=1e-9) and not torch.allclose(a[11], c[11], atol=1e-9) and torch.allclose(a[12:], c[12:], atol=1e-9)
    g = torch.Generator().manual_seed(5)
    T, H, G, d, dv = 9, 4, 2, 6, 5
    q, k, v = (torch.randn(T, n, m, generator=g, dtype=torch.float64) for n, m in ((H, d), (G, d), (G, dv)))
    plain = D.mixed_head_softmax_rows(q, k, v, 0.7, torch.eye(H, dtype=torch.float64))
    for h in range(H):
        p = torch.softmax(0.7 * (k[:, h // 2] @ q[8, h]), -1)
        assert torch.allclose(plain[8, h], p @ v[:, h // 2], atol=1e-12)
    talk = torch.randn(H, H, generator=g, dtype=torch.float64)
    mixed = D.mixed_head_softmax_rows(q, k, v, 0.7, talk)
    folded_q = torch.stack([torch.cat([sum(talk[h, gg] * q[:, gg] for gg in range(c * 2, c * 2 + 2)) for c in range(G)], -1) for h in range(H)], 1)   # [T, H, G * d]
    s = 0.7 * torch.einsum("hx,sx->hs", folded_q[8], k.reshape(T, G * d))
    for h in range(H):
        assert torch.allclose(mixed[8, h], torch.softmax(s[h], -1) @ v[:, h // 2], atol=1e-12)
    z = torch.tensor([[0.1, 2.0, -1.0, 2.0, 0.5]], dtype=torch.float64)
    sel, w = D.route(z, 3)
    assert sel.tolist() == [[1, 3, 4]] and abs(float(w.sum()) - 1.0) < 1e-12 and abs(float(w[0, 0] / w[0, 2]) - math.exp(1.5)) < 1e-9
    assert abs(float(D.xielu(torch.tensor([2.0], dtype=torch.float64), 0.0, 0.0)) - (math.log(2.0) * 4 + 1)) < 1e-12
