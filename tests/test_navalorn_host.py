"""What the Navalorn decoder decides on the host: its configuration, the layers it is built from and the order they run
in, the cache it asks for; and the plain implementation's own properties (the oracle is checked apart from the code it
judges)."""
import math

import numpy as np
import pytest
import torch

import ghost_infer_b200 as gi
import plain_navalorn as pn
from ghost_infer_b200.cache.sequence_cache import CacheRequest, SequenceCache
from ghost_infer_b200.config import ConfigError, architecture_of, parse_config
from ghost_infer_b200.engine.model import Model

MIX = {"heads": 3, "dim": 10, "rot_dim": 6, "vdim": 12, "kv_rank": 20, "q_rank": 14, "scale": 0.2,
       "rot": {"base": 5000.0, "dims": 4, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}}}
MOE = {"kind": "moe", "router": {"experts": 4, "top": 2}, "expert": {"ff": 8}}
CFG = {"architecture": "Navalorn", "width": 32, "vocab": 50, "norm": {"eps": 1e-6}, "layers": [
    {"type": "latent_attention", "mixer": MIX, "mlp": {"kind": "dense", "ff": 40}},
    {"type": "latent_attention", "mixer": MIX, "mlp": MOE},
    {"type": "latent_attention", "mixer": MIX, "mlp": MOE, "weights_of": 1},
    {"type": "latent_attention", "mixer": dict(MIX, heads=1), "mlp": None},
    {"type": "latent_attention", "mixer": MIX, "mlp": {"kind": "dense", "ff": 40}, "weights_of": 0},
]}


def test_configuration_is_typed_and_checked():
    assert architecture_of(CFG) == "Navalorn"
    cfg = parse_config(CFG)
    assert cfg.width == 32 and cfg.vocab_size == 50 and cfg.num_hidden_layers == 5 and cfg.norm_eps == 1e-6
    assert cfg.layers[3].mlp is None and cfg.layers[2].weights_of == 1 and cfg.layers[1].mlp.top == 2
    assert cfg.layers[0].mixer.rot.scaling.original == 64 and cfg.max_position_embeddings == 256
    layer = lambda **kw: dict(CFG["layers"][0], **kw)
    for bad in (dict(CFG, layers=[]), dict(CFG, layers=[layer(type="attention")]),
                dict(CFG, layers=[layer(mixer=dict(MIX, rot=dict(MIX["rot"], dims=8)))]),          # more numbers turn than the part has
                dict(CFG, layers=[layer(mixer=dict(MIX, rot=dict(MIX["rot"], dims=3)))]),
                dict(CFG, layers=[layer(mixer={k: v for k, v in MIX.items() if k != "kv_rank"})]),
                dict(CFG, layers=[layer(mlp={"kind": "moe", "router": {"experts": 2, "top": 3}, "expert": {"ff": 4}})]),
                dict(CFG, layers=[layer(mlp={"kind": "gated", "ff": 4})]),
                dict(CFG, layers=[layer(), layer(weights_of=1)]), dict(CFG, layers=[layer(), layer(weights_of=5)]),
                dict(CFG, layers=[layer(), layer(weights_of=0, mlp=None)]),                           # other sizes than the lender's
                {k: v for k, v in CFG.items() if k != "norm"}):
        with pytest.raises(ConfigError):
            parse_config(bad)


def test_layers_are_put_together_from_the_configuration():
    model = Model.from_config_dict(CFG)
    assert [e.layer for e in model.spec.schedule] == [0, 1, 1, 2, 0] and all(e.memory_of is None for e in model.spec.schedule)
    assert [type(l.block.mixer).__name__ for l in model.layers] == ["LatentAttention"] * 3
    assert [type(l.block.ffn).__name__ for l in model.layers] == ["Mlp", "ScoredExperts", "NoneType"]
    assert type(model.embedding_norm).__name__ == "LayerNorm" and type(model.final_norm).__name__ == "LayerNorm" and model.head.tied
    names = {w.name: tuple(w.shape) for w in model.weight_manifest()}
    assert names["l0.mix.dq"] == (14, 32) and names["l0.mix.uq"] == (3 * 16, 14) and names["l0.mix.dkv"] == (26, 32)
    assert names["l0.mix.uk"] == (30, 20) and names["l0.mix.uv"] == (36, 20) and names["l0.mix.o"] == (32, 36)
    assert names["l0.mlp.up.b"] == (40,) and names["l0.mlp.down.b"] == (32,) and names["l1.mlp.e3.down"] == (32, 8)
    assert names["l3.mix.uq"] == (16, 14) and "l3.norm2" not in names and "l2.norm1" not in names and "l4.mix.o" not in names
    assert names["embed.norm"] == (32,) and "head" not in names
    assert set(names) == set(pn.random_weights(CFG))
    reqs = model.memory_requests()
    assert len(reqs) == 5 and all(r[1] == CacheRequest("full", 1, 26, None, 20, values_in_keys=True) and r[2] is None for r in reqs[:3])
    mixer = model.layers[0].block.mixer
    assert mixer.rot == 4 and mixer.position.pairing == "adjacent" and abs(mixer.position.magnitude - (0.1 * math.log(4.0) + 1)) < 1e-12
    f, mag = pn.rotary_frequencies(4, 5000.0, MIX["rot"]["scaling"])
    assert np.allclose(mixer.position.inv_freq_host.double().numpy(), f, rtol=1e-6)


def test_a_latent_cache_stores_one_row_per_position_and_no_values():
    req = CacheRequest("full", 1, 26, None, 20, values_in_keys=True)
    cache = SequenceCache([(0, req, None, None), (1, req, None, None)], max_tokens=64 * 4, max_slots=2, max_seq_len=1000, dtype=torch.bfloat16)
    mem = cache.memory(1)
    assert tuple(mem.k.shape[1:]) == (1, 64, 26) and mem.v is None and mem.writes
    assert cache.bytes_per_token() == 2 * 26 * 2
    assert cache.memory(0).k.data_ptr() != mem.k.data_ptr()            # every run of a layer has rows of its own
    s = cache.open_slot()
    cache.reserve([(s, 130)])
    cache.commit(s, 130)
    assert cache.free_pages == cache.n_pages - 3
    cache.close_slot(s)
    assert cache.free_pages == cache.n_pages
    with pytest.raises(ValueError):
        CacheRequest("full", 1, 8, None, 9, values_in_keys=True)


# ---- the plain implementation's own properties ---------------------------------------------------------------------
def test_plain_model_is_causal_and_borrowed_layers_have_caches_of_their_own():
    w = pn.random_weights(CFG, seed=1)
    t = np.random.default_rng(0).integers(0, 50, size=40).tolist()
    full, layers = pn.forward(CFG, w, t, return_layers=True)
    assert layers.shape == (5, 40, 32)
    assert np.allclose(pn.forward(CFG, w, t[:25]), full[:25], rtol=0, atol=1e-12)
    t2 = list(t)
    t2[30] = (t2[30] + 1) % 50
    b = pn.forward(CFG, w, t2)
    assert np.allclose(b[:30], full[:30], rtol=0, atol=1e-12) and np.abs(b[30:] - full[30:]).max() > 1e-6
    # the second run of a layer is not a copy of the first: its input differs, so does what it adds
    assert np.abs((layers[2] - layers[1]) - (layers[1] - layers[0])).max() > 1e-3


def test_plain_mechanisms_on_small_cases_worked_by_hand():
    # layer norm of (1, 3): mean 2, variance 1
    assert np.allclose(pn.layer_norm(np.array([[1.0, 3.0]]), np.array([2.0, 0.5]), 0.0), [[-2.0, 0.5]])
    assert np.allclose(pn.rms_norm(np.array([[3.0, 4.0]]), np.array([1.0, 1.0]), 0.0), [[3.0 / math.sqrt(12.5), 4.0 / math.sqrt(12.5)]])
    # a quarter turn of the pair (1, 0) at position 1 with frequency pi / 2, stretched by 1.5: (0, 1.5)
    out = pn.rotate_pairs(np.array([[1.0, 0.0]]), [1], np.array([math.pi / 2]), 1.5)
    assert np.allclose(out, [[0.0, 1.5]], atol=1e-12)
    # frequencies: 8 numbers, base 100, 64 positions stretched 4 times, ramp from 4 turns to 1 turn (pair indices 0.81 and
    # 2.02: lo 0, hi 3): the ramp is 0, 1/3, 2/3, 1
    f, mag = pn.rotary_frequencies(8, 100.0, {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 1.0})
    plain = [100.0 ** (-2 * i / 8) for i in range(4)]
    assert np.allclose(f, [plain[0], plain[1] * (1 / 12 + 2 / 3), plain[2] * (1 / 6 + 1 / 3), plain[3] / 4]) and abs(mag - (0.1 * math.log(4) + 1)) < 1e-12
    assert pn.rotary_frequencies(8, 100.0, None)[1] == 1.0
    # router: of the products (1, 3, 2) the largest two are experts 1 and 2, weighted sigmoid(3) and sigmoid(2) as they are;
    # the weight goes onto the input: down * relu(up * (w * h))^2
    ids, wts = pn.route(np.array([[1.0]]), np.array([[1.0], [3.0], [2.0]]), 2)
    sg = lambda z: 1 / (1 + math.exp(-z))
    assert ids.tolist() == [[1, 2]] and np.allclose(wts, [[sg(3), sg(2)]])
    wr = {"router": np.array([[1.0], [3.0], [2.0]])}
    for e, u in enumerate((5.0, 2.0, -1.0)):
        wr.update({f"e{e}.up": np.array([[u]]), f"e{e}.down": np.array([[3.0]])})
    assert np.allclose(pn.routed_feed_forward(np.array([[1.0]]), wr, 3, 2), 3.0 * (2.0 * sg(3)) ** 2 + 0.0)
    assert np.allclose(pn.dense_feed_forward(np.array([[2.0]]), {"up": np.array([[1.0], [-1.0]]), "up.b": np.array([1.0, 1.0]),
                                                               "down": np.array([[1.0, 1.0]]), "down.b": np.array([0.5])}), [[9.5]])


def test_command_line_makes_and_lists_a_model_folder(tmp_path, capsys):
    import json
    from ghost_infer_b200 import cli
    from ghost_infer_b200.weights.safetensors_io import SafetensorsFile
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(CFG))
    out = tmp_path / "model"
    assert cli.main(["random", str(cfg_file), str(out), "--seed", "3"]) == 0
    names = set(SafetensorsFile(str(out / "model.safetensors")).names())
    assert names == {w.name for w in Model.from_config_dict(CFG).weight_manifest()}
    assert cli.main(["inspect", str(out)]) == 0
    text = capsys.readouterr().out
    assert "l0.mix.dkv.norm" in text and "embed.norm" in text and f"{len(names)} tensors" in text
    # the file written by the test's own writer binds too
    w = pn.random_weights(CFG, seed=4)
    other = tmp_path / "other"
    other.mkdir()
    (other / "config.json").write_text(json.dumps(CFG))
    pn.write_bf16_file(str(other / "model.safetensors"), w)
    from ghost_infer_b200.weights.loader import load_model_tensors
    model = Model.from_config_dict(CFG)
    got = load_model_tensors(str(other), model.weight_manifest(), model.ignorable_tensors())
    assert torch.equal(got["l0.mix.dq"].float(), torch.from_numpy(w["l0.mix.dq"]).float())
