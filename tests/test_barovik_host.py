"""What the Barovik decoder decides on the host: its configuration, the layers it is built from, the cache it asks
for; and the plain implementation's own properties (the oracle is checked apart from the code it judges)."""
import numpy as np
import pytest
import torch

import ghost_infer_b200 as gi
import plain_barovik as pb
from ghost_infer_b200.cache.sequence_cache import CacheRequest, SequenceCache
from ghost_infer_b200.config import ConfigError, architecture_of, parse_config
from ghost_infer_b200.engine.model import Model

ATT = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.25, "softcap": 30.0, "mask": {"size": 20}, "v_mix": True}
SSM = {"heads": 2, "vdim": 8, "state": 4, "groups": 1, "conv": 3, "norm_groups": 2}
CFG = {"architecture": "Barovik", "width": 32, "vocab": 50, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6}, "layers": [
    {"type": "mamba2", "mixer": SSM, "mlp": None},
    {"type": "attention", "mixer": ATT, "mlp": {"kind": "dense", "ff": 40}},
    {"type": "attention", "mixer": dict(ATT, v_mix=False), "mlp": {"kind": "moe", "router": {"experts": 4, "top": 2}, "expert": {"ff": 8}}},
    {"type": "attention", "mixer": ATT, "mlp": {"kind": "moe", "router": {"experts": 3, "top": 1}, "expert": {"ff": 8}, "shared": {"ff": 12}}},
]}


def test_the_architecture_is_found_by_its_single_name():
    assert architecture_of(CFG) == "Barovik"
    assert architecture_of({"architectures": ["LlamaForCausalLM"], "architecture": "x"}) == "LlamaForCausalLM"
    with pytest.raises(ConfigError):
        architecture_of({"width": 3})


def test_configuration_is_typed_and_checked():
    cfg = parse_config(CFG)
    assert cfg.width == 32 and cfg.vocab_size == 50 and cfg.num_hidden_layers == 4 and cfg.embedding_scale == 2.0
    assert cfg.layers[0].mlp is None and cfg.layers[1].mixer.chunk == 20 and cfg.layers[3].mlp.shared_ff == 12
    for bad in (dict(CFG, layers=[]), dict(CFG, layers=[{"type": "conv", "mixer": {}}]),
                dict(CFG, layers=[{"type": "attention", "mixer": dict(ATT, heads=3)}]),
                dict(CFG, layers=[{"type": "mamba2", "mixer": dict(SSM, groups=3)}]),
                dict(CFG, layers=[{"type": "mamba2", "mixer": dict(SSM, norm_groups=3)}]),
                dict(CFG, layers=[{"type": "mamba2", "mixer": SSM, "mlp": {"kind": "moe", "router": {"experts": 2, "top": 3}, "expert": {"ff": 4}}}]),
                {k: v for k, v in CFG.items() if k != "norm"}):
        with pytest.raises(ConfigError):
            parse_config(bad)


def test_layers_are_put_together_from_the_configuration():
    model = Model.from_config_dict(CFG)
    mixers = [layer.block.mixer for layer in model.layers]
    assert [type(m).__name__ for m in mixers] == ["Mamba2", "SinkAttention", "SinkAttention", "SinkAttention"]
    assert [getattr(m, "value_mix", None) for m in mixers] == [None, "source", None, "blend"]
    assert model.layers[0].block.ffn is None and model.layers[0].block.ffn_norm is None
    names = {w.name: tuple(w.shape) for w in model.weight_manifest()}
    assert names["l0.mix.in"] == (2 * 16 + 2 * 4 + 2, 32) and names["l0.mix.conv"] == (24, 3)
    assert names["l1.mix.v"] == (16, 32) and names["l1.mix.o"] == (32, 32) and names["l1.mix.vmix"] == ()
    assert "l2.mix.vmix" not in names and "l0.norm2" not in names and names["l3.mlp.shared.sg"] == (1, 32)
    assert names["embed"] == (50, 32) and names["head"] == (50, 32) and names["final.norm"] == (32,)
    assert set(names) == set(pb.random_weights(CFG))
    reqs = model.memory_requests()
    assert reqs[0][1] is None and reqs[0][2].shape == (2 * 4 * 8 + 2 * 24,)
    assert reqs[1][1] == CacheRequest("chunk", 2, 16, 20, 8) and reqs[1][2] is None


def test_a_chunk_cache_keeps_the_newest_chunk_and_values_of_their_own_width():
    req = CacheRequest("chunk", 2, 16, 100, 8)
    cache = SequenceCache([(0, req, None, None)], max_tokens=64 * 4, max_slots=2, max_seq_len=10000, dtype=torch.float32)
    mem = cache.memory(0)
    assert tuple(mem.k.shape[1:]) == (2, 64, 16) and tuple(mem.v.shape[1:]) == (2, 64, 8) and mem.chunk == 100 and mem.window is None
    assert cache.bytes_per_token() == 2 * (16 + 8) * 4
    s = cache.open_slot()
    at = 0
    for n in (99, 1, 1, 100, 50, 60, 100, 100, 100, 100, 100):          # 811 tokens through a pool of four pages
        cache.reserve([(s, at + n)])
        at += n
        cache.commit(s, at)
        first_needed = (at // 100 * 100) // 64   # the page that holds the start of the chunk position `at` lies in
        g = cache.groups[0]
        assert g.first_live[s] == first_needed
        assert all(p == 0 for p in g.pages[s][:first_needed]) and all(p > 0 for p in g.pages[s][first_needed:])
    assert cache.truncate(s, 10) == at            # what was given back cannot be rewound
    cache.close_slot(s)
    assert cache.free_pages == cache.n_pages
    with pytest.raises(ValueError):
        CacheRequest("chunk", 1, 8)


# ---- the plain implementation's own properties ---------------------------------------------------------------------
def test_plain_model_is_causal_and_its_chunks_are_closed():
    w = pb.random_weights(CFG, seed=1)
    t = np.random.default_rng(0).integers(0, 50, size=47).tolist()
    full = pb.forward(CFG, w, t)
    assert np.allclose(pb.forward(CFG, w, t[:30]), full[:30], rtol=0, atol=1e-12)
    # an attention-only model: a token before a chunk's start does not reach a query inside the chunk
    only = dict(CFG, layers=[CFG["layers"][1]])
    w1 = pb.random_weights(only, seed=2)
    a = pb.forward(only, w1, t)
    t2 = list(t)
    t2[19] = (t2[19] + 1) % 50
    b = pb.forward(only, w1, t2)
    assert np.abs(a[19] - b[19]).max() > 1e-6 and np.allclose(a[20:], b[20:], rtol=0, atol=1e-12) and np.allclose(a[:19], b[:19])


def test_plain_mechanisms_on_small_cases_worked_by_hand():
    # convolution: taps (1, 2, 3) over inputs 1, 1, 1 with zeros before the start
    out = pb.causal_conv(np.ones((3, 1)), np.array([[1.0, 2.0, 3.0]]), np.array([0.5]))
    assert out[:, 0].tolist() == [3.5, 5.5, 6.5]
    # recurrence with one head, one state row, one column: S_t = a S_(t-1) + dt B x, y = S C + D x
    y = pb.ssm_scan(np.ones((2, 1, 1)), np.full((2, 1, 1), 2.0), np.full((2, 1, 1), 3.0), np.full((2, 1), 0.5),
                    np.array([0.0]), np.array([10.0]), 1, 1)
    a = np.exp(-0.5)
    assert np.allclose(y[:, 0, 0], [3.0 * 1.0 + 10.0, 3.0 * (a * 1.0 + 1.0) + 10.0])
    # a sink as large as the only score halves the weight of the only key
    m = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "scale": 1.0}
    wts = {"q": np.array([[1.0]]), "k": np.array([[1.0]]), "v": np.array([[1.0]]), "o": np.array([[1.0]]), "sink": np.array([4.0])}
    out, _ = pb.sink_attention(np.array([[2.0]]), wts, m)
    assert np.allclose(out, [[1.0]])
    # router: the two largest of (1, 3, 2) are experts 1 and 2 with weights softmax(3, 2)
    mlp = {"router": {"experts": 3, "top": 2}}
    wr = {"router": np.array([[1.0], [3.0], [2.0]])}
    for e, g in enumerate((5.0, 1.0, 2.0)):
        wr.update({f"e{e}.gate": np.array([[g]]), f"e{e}.up": np.array([[1.0]]), f"e{e}.down": np.array([[1.0]])})
    p = np.exp([3.0, 2.0]) / np.exp([3.0, 2.0]).sum()
    assert np.allclose(pb.routed_ff(np.array([[1.0]]), wr, mlp), p[0] * pb.silu(1.0) + p[1] * pb.silu(2.0))
    assert abs(pb.gelu_tanh(np.array(1.0)) - 0.8411919906) < 1e-9


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
    assert "l0.mix.A_log" in text and f"{len(names)} tensors" in text
    # a file may carry tensors for what the configuration switches off; anything else is refused
    from ghost_infer_b200.weights.loader import WeightsError, load_model_tensors
    model = Model.from_config_dict(CFG)
    assert "l2.mix.vmix" in model.ignorable_tensors() and "l0.norm2" in model.ignorable_tensors()
    load_model_tensors(str(out), model.weight_manifest(), model.ignorable_tensors())
    with pytest.raises(WeightsError):
        load_model_tensors(str(out), [w for w in model.weight_manifest() if w.name != "head"], model.ignorable_tensors())
