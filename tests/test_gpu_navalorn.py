"""The Navalorn decoder through the engine, against the plain implementation (`plain_navalorn.py`).

Every test makes its own small configuration and random weights.  The configurations differ from each other in every
size and constant and exercise the values that are easily 1 or equal: one head and many, a latent narrower and wider than
a head, a rotated part of which only some numbers turn, no rotated part's scaling at all, a scaling factor of 1, one
expert chosen and all of them, a layer without feed-forward, layers that borrow another layer's tensors (one after the
other and with a layer of their own between), sizes that are multiples of 8 (the tensor-core kernels) and sizes that are
not (the plain ones).  Scores are made sharp (the queries' up-projection scaled up) so that a key one position off, or a
rotation by the wrong angle, moves the logits by far more than the tolerance.
"""
import json
import os

import numpy as np
import pytest
import torch

import ghost_infer_b200 as gi
import plain_navalorn as pn

pytestmark = pytest.mark.gpu


def mixer(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot_dims=None, base=10000.0, scaling=(4.0, 64, 8.0, 1.0)):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}
    if rot_dim:
        m["rot"] = {"base": base, "dims": rot_dims or rot_dim}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return m


def moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(m, mlp, weights_of=None):
    out = {"type": "latent_attention", "mixer": m, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def model_cfg(width, vocab, layers, eps=1e-5):
    return {"architecture": "Navalorn", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}


M_A = mixer(4, 16, 8, 24, 40, 32, 0.25)                                  # multiples of 8: the tensor-core kernels in 16 bits
M_A2 = mixer(3, 24, 16, 8, 64, 48, 0.2, rot_dims=8, base=500.0, scaling=(16.0, 16, 4.0, 0.5))
CFG_A = model_cfg(96, 200, [
    layer(M_A, dense(136)),
    layer(M_A2, moe(6, 2, 40)),
    layer(M_A2, moe(6, 2, 40), weights_of=1),
    layer(M_A, None),
    layer(M_A2, moe(6, 2, 40), weights_of=2),
    layer(M_A, dense(136), weights_of=0),
])
M_B = mixer(5, 12, 6, 10, 21, 13, 0.35, rot_dims=4, base=77.0, scaling=None)        # nothing a multiple of 8: the plain kernels
M_B2 = mixer(1, 20, 2, 36, 9, 50, 0.3, scaling=(1.0, 32, 2.0, 1.0))
CFG_B = model_cfg(80, 301, [
    layer(M_B, moe(3, 3, 32)),
    layer(M_B2, dense(72)),
    layer(M_B, moe(3, 3, 32), weights_of=0),
], eps=3e-6)
# for the bfloat16 path every expert is chosen: what a token gets is then a continuous function of the router's products,
# and a near tie that the rounding of activations decides the other way does not send the token elsewhere
CFG_A16 = json.loads(json.dumps(CFG_A))
for _l in CFG_A16["layers"]:
    if _l["mlp"] and _l["mlp"]["kind"] == "moe":
        _l["mlp"]["router"]["top"] = _l["mlp"]["router"]["experts"]
# twenty heads (more than one tensor-core tile of rows holds per token in a one-token step's keys mode), a wide latent
CFG_C = model_cfg(128, 150, [
    layer(mixer(20, 8, 8, 16, 136, 24, 0.3), dense(96)),
    layer(mixer(2, 32, 32, 32, 264, 64, 0.15, rot_dims=32, scaling=(8.0, 128, 32.0, 1.0)), moe(4, 4, 32)),
])
CONFIGS = {"A": CFG_A, "A16": CFG_A16, "B": CFG_B, "C": CFG_C}
_made = {}


def made(name):
    if name not in _made:
        cfg = CONFIGS[name]
        w = pn.random_weights(cfg, seed=len(name) + ord(name[0]))
        for k in w:
            if name in ("A", "B") and k.endswith("mix.uq"):
                w[k] = w[k] * 2.0               # sharp scores (exactly representable: a power of two)
        _made[name] = (cfg, w, {k: torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16) for k, v in w.items()})
    return _made[name]


def engine_for(name, dtype, max_tokens=64 * 40, max_slots=None):
    cfg, _, tensors = made(name)
    model = gi.Model.from_config_dict(cfg).bind(tensors, dtype, "cuda:0")
    cache = model.new_cache(max_tokens=max_tokens, max_seq_len=4096, max_slots=max_slots, beyond_trained_positions=True)
    return gi.Engine(model, cache)


_plain = {}


def plain(name, tokens):
    key = (name, tuple(tokens))
    if key not in _plain:
        cfg, w, _ = made(name)
        _plain[key] = pn.forward(cfg, w, list(tokens))
    return _plain[key]


def toks(name, n, seed):
    return np.random.default_rng(seed).integers(0, CONFIGS[name]["vocab"], size=n).tolist()


def check(got, ref, dtype, what=""):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    scale = max(1.0, float(np.abs(ref).max()))
    err = np.abs(got - ref)
    if dtype == "float32":
        assert err.max() <= 5e-5 * scale, f"{what}: max error {err.max():.3e} (scale {scale:.2f}) at {np.unravel_index(err.argmax(), err.shape)}"
    else:
        rms = float(np.sqrt((err ** 2).mean()))
        assert err.max() <= 0.08 * scale and rms <= 0.012 * scale, f"{what}: max {err.max():.3e} rms {rms:.3e} (scale {scale:.2f})"


def run_whole(eng, tokens):
    s = eng.cache.open_slot()
    out = eng.step([gi.StepEntry(s, tokens, list(range(len(tokens))))]).cpu().numpy()
    eng.cache.close_slot(s)
    return out


PATHS = [("A", "float32"), ("B", "float32"), ("C", "float32"), ("A16", "bfloat16"), ("C", "bfloat16")]

# ---- each mechanism alone: one-layer models --------------------------------------------------------------------------
ALONE = {
    "attention": layer(mixer(3, 8, 4, 12, 20, 16, 0.4), None),
    "attention_rotation_only": layer(mixer(2, 1, 16, 8, 8, 8, 0.5, base=50.0), None),
    "attention_no_rotation": layer(mixer(2, 16, 0, 8, 24, 8, 0.3), None),
    "dense": layer(mixer(1, 4, 2, 4, 4, 4, 0.5), dense(52)),
    "moe_one_of_many": layer(mixer(1, 4, 2, 4, 4, 4, 0.5), moe(7, 1, 20)),
    "moe_three": layer(mixer(1, 4, 2, 4, 4, 4, 0.5), moe(7, 3, 20)),
}


@pytest.mark.parametrize("which", sorted(ALONE))
def test_each_mechanism_alone(which):
    cfg = model_cfg(48, 90, [ALONE[which]])
    w = pn.random_weights(cfg, seed=11)
    tensors = {k: torch.from_numpy(np.asarray(v, dtype=np.float32)) for k, v in w.items()}
    model = gi.Model.from_config_dict(cfg).bind(tensors, "float32", "cuda:0")
    eng = gi.Engine(model, model.new_cache(max_tokens=256, max_seq_len=256, beyond_trained_positions=True))
    t = np.random.default_rng(5).integers(0, 90, size=70).tolist()
    check(run_whole(eng, t), pn.forward(cfg, w, t), "float32", which)


def test_embedding_norm_and_tied_head_alone():
    """One layer whose output projection and feed-forward are zero: the logits are the normed embedding, normed again,
    against the embedding table."""
    cfg = model_cfg(40, 60, [layer(mixer(2, 4, 2, 4, 8, 8, 0.5), None)])
    w = pn.random_weights(cfg, seed=2)
    w["l0.mix.o"] = w["l0.mix.o"] * 0
    tensors = {k: torch.from_numpy(np.asarray(v, dtype=np.float32)) for k, v in w.items()}
    model = gi.Model.from_config_dict(cfg).bind(tensors, "float32", "cuda:0")
    eng = gi.Engine(model, model.new_cache(max_tokens=128, max_seq_len=128))
    t = list(range(0, 60, 7))
    x = pn.layer_norm(pn.layer_norm(w["embed"][t], w["embed.norm"], 1e-5), w["final.norm"], 1e-5) @ w["embed"].T
    check(run_whole(eng, t), x, "float32")


# ---- whole prompts, decoding, portions, batches -----------------------------------------------------------------------
@pytest.mark.parametrize("name,dtype", PATHS)
def test_whole_prompt(name, dtype):
    eng = engine_for(name, dtype)
    for n, seed in ((1, 1), (2, 2), (64, 3), (65, 4), (200, 5)):
        t = toks(name, n, seed)
        check(run_whole(eng, t), plain(name, t), dtype, f"{name} {n} tokens")


@pytest.mark.parametrize("name,dtype", PATHS)
@pytest.mark.parametrize("graph", [False, True])
def test_prompt_then_token_by_token(name, dtype, graph):
    eng = engine_for(name, dtype)
    t = toks(name, 150, 21)
    s = eng.cache.open_slot()
    rows = [eng.step([gi.StepEntry(s, t[:60], list(range(60)))]).cpu().numpy()]
    run = eng.decoder([s], use_graph=graph)
    for i in range(60, len(t)):          # across the page borders at 64 and 128
        rows.append(run.forward(tokens=[t[i]]).cpu().numpy().copy())
    eng.cache.close_slot(s)
    check(np.concatenate(rows, 0), plain(name, t), dtype)


def test_decoding_from_the_first_token():
    eng = engine_for("B", "float32")
    t = toks("B", 70, 8)
    s = eng.cache.open_slot()
    rows = [eng.step([gi.StepEntry(s, [x], [0])]).cpu().numpy() for x in t]
    eng.cache.close_slot(s)
    check(np.concatenate(rows, 0), plain("B", t), "float32")


@pytest.mark.parametrize("name,dtype", PATHS)
def test_portions_of_several_sizes(name, dtype):
    eng = engine_for(name, dtype)
    t = toks(name, 140, 31)
    ref = plain(name, t)
    for cuts in ((2, 4, 66, 130, 140), (63, 64, 65, 128, 140), (1, 3, 140)):
        s = eng.cache.open_slot()
        rows, a = [], 0
        for b in cuts:
            rows.append(eng.step([gi.StepEntry(s, t[a:b], list(range(b - a)))]).cpu().numpy())
            a = b
        eng.cache.close_slot(s)
        check(np.concatenate(rows, 0), ref, dtype, f"{name} cut at {cuts}")


def test_float32_does_not_depend_on_the_cut_or_the_batch():
    eng = engine_for("A", "float32")
    t, other = toks("A", 100, 41), toks("A", 37, 42)
    whole = run_whole(eng, t)
    s = eng.cache.open_slot()
    cut = np.concatenate([eng.step([gi.StepEntry(s, t[a:b], list(range(b - a)))]).cpu().numpy() for a, b in ((0, 7), (7, 71), (71, 100))], 0)
    eng.cache.close_slot(s)
    assert np.array_equal(whole, cut)
    s1, s2 = eng.cache.open_slot(), eng.cache.open_slot()
    both = eng.step([gi.StepEntry(s2, other, [0]), gi.StepEntry(s1, t, list(range(100)))]).cpu().numpy()
    eng.cache.close_slot(s1); eng.cache.close_slot(s2)
    assert np.array_equal(whole, both[1:])


@pytest.mark.parametrize("name,dtype", PATHS)
def test_unequal_batch_against_each_alone(name, dtype):
    eng = engine_for(name, dtype)
    prompts = [toks(name, n, 50 + n) for n in (90, 3, 66, 1, 130)]
    tails = 6
    slots = [eng.cache.open_slot() for _ in prompts]
    cut = [max(1, len(p) - tails) for p in prompts]
    out = eng.step([gi.StepEntry(s, p[:c], list(range(c))) for s, p, c in zip(slots, prompts, cut)]).cpu().numpy()
    got = [[out[sum(cut[:i]):sum(cut[:i + 1])]] for i in range(len(prompts))]
    live = list(range(len(prompts)))
    fed = list(cut)
    while live:
        live = [i for i in live if fed[i] < len(prompts[i])]
        if not live:
            break
        run = eng.decoder([slots[i] for i in live])          # the shorter requests end earlier
        rows = run.forward(tokens=[prompts[i][fed[i]] for i in live]).cpu().numpy()
        for k, i in enumerate(live):
            got[i].append(rows[k:k + 1].copy())
            fed[i] += 1
    for s in slots:
        eng.cache.close_slot(s)
    for i, p in enumerate(prompts):
        check(np.concatenate(got[i], 0), plain(name, p), dtype, f"{name}: request {i} of the batch")


def test_slots_and_pages_used_again():
    eng = engine_for("A", "float32", max_tokens=64 * 6, max_slots=2)
    free = eng.cache.free_pages
    for round_ in range(4):
        a, b = toks("A", 100 + round_, 60 + round_), toks("A", 30, 70 + round_)
        sa, sb = eng.cache.open_slot(), eng.cache.open_slot()
        out = eng.step([gi.StepEntry(sa, a, [len(a) - 1]), gi.StepEntry(sb, b, [len(b) - 1])]).cpu().numpy()
        check(out[0:1], plain("A", a)[-1:], "float32", f"round {round_}")
        check(out[1:2], plain("A", b)[-1:], "float32", f"round {round_}")
        eng.cache.close_slot(sb)
        sc = eng.cache.open_slot()                       # the slot and the pages b just gave back
        c = toks("A", 70, 90 + round_)
        check(eng.step([gi.StepEntry(sc, c, [len(c) - 1])]).cpu().numpy(), plain("A", c)[-1:], "float32")
        eng.cache.close_slot(sa); eng.cache.close_slot(sc)
        assert eng.cache.free_pages == free


# ---- keys far away, the first tokens, and a position that is one off ---------------------------------------------------
def far_key_model():
    """One layer whose weights are set so that token 1's queries find token 0's keys: with h_0 and h_1 the mixer's inputs
    for the two tokens, the queries' down-projection is the keys' times h_0 h_1^T / |h_1|^2 (so that token 1's query
    latent is token 0's latent), both latents share a norm weight, every head's unrotated query part uses the keys'
    up-projection and the rotated query part is zero: q_1 . k_0 = |W_uk c_0|^2, and with a scale of 4 the softmax is sharp."""
    cfg = model_cfg(32, 64, [layer(mixer(2, 8, 8, 8, 16, 16, 4.0, base=10000.0, scaling=None), None)])
    w = pn.random_weights(cfg, seed=5)
    h = pn.layer_norm(pn.layer_norm(w["embed"][:2], w["embed.norm"], 1e-5), w["l0.norm1"], 1e-5)
    w["l0.mix.dq"] = pn._to_bf16_values(w["l0.mix.dkv"][:16] @ np.outer(h[0], h[1]) / (h[1] @ h[1])).astype(np.float64)
    w["l0.mix.dq.norm"] = w["l0.mix.dkv.norm"].copy()
    uq = w["l0.mix.uq"].reshape(2, 16, 16)
    uq[:, :8, :] = w["l0.mix.uk"].reshape(2, 8, 16)
    uq[:, 8:, :] = 0.0
    w["l0.mix.uq"] = uq.reshape(32, 16)
    return cfg, w


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds(dtype):
    """Token 0 at position 3, token 1 at the very end of 400 tokens that are neither: the last position looks at
    position 3 across six page borders; a kernel that loses far keys, or a page, misses by far more than the tolerance."""
    cfg, w = far_key_model()
    tensors = {k: torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16) for k, v in w.items()}
    model = gi.Model.from_config_dict(cfg).bind(tensors, dtype, "cuda:0")
    eng = gi.Engine(model, model.new_cache(max_tokens=64 * 16, max_seq_len=1024, beyond_trained_positions=True))
    r = np.random.default_rng(9)
    t = r.integers(2, 64, size=400).tolist()
    t[3], t[-1] = 0, 1
    ref = pn.forward(cfg, w, t)
    check(run_whole(eng, t)[-40:], ref[-40:], dtype, "whole")
    s = eng.cache.open_slot()
    eng.step([gi.StepEntry(s, t[:380], [])])
    run = eng.decoder([s])
    rows = [run.forward(tokens=[x]).cpu().numpy().copy() for x in t[380:]]
    eng.cache.close_slot(s)
    check(np.concatenate(rows, 0), ref[380:], dtype, "decoded")
    # and the far key matters: without it the last logits are others
    t2 = list(t)
    t2[3] = 5
    assert np.abs(pn.forward(cfg, w, t2)[-1] - ref[-1]).max() > 0.05 * np.abs(ref[-1]).max()


def test_positions_count_from_zero_in_each_sequence():
    """Two requests with the same tokens in one batch, and the same request after others used the slot: the same logits,
    because angles follow the position in the sequence, not the place in the batch or the cache."""
    eng = engine_for("B", "float32")
    t = toks("B", 50, 3)
    ref = plain("B", t)
    s0, s1, s2 = (eng.cache.open_slot() for _ in range(3))
    out = eng.step([gi.StepEntry(s0, toks("B", 20, 4), []), gi.StepEntry(s1, t, list(range(50))), gi.StepEntry(s2, t, list(range(50)))]).cpu().numpy()
    for s in (s0, s1, s2):
        eng.cache.close_slot(s)
    check(out[:50], ref, "float32")
    assert np.array_equal(out[:50], out[50:])


def test_long_decoding_through_the_graph_runner():
    """330 decoded tokens: length buckets, five page borders, more slices as the context grows."""
    eng = engine_for("A16", "bfloat16")
    t = toks("A16", 340, 71)
    s = eng.cache.open_slot()
    rows = [eng.step([gi.StepEntry(s, t[:10], list(range(10)))]).cpu().numpy()]
    run = eng.decoder([s])
    for i in range(10, len(t)):
        rows.append(run.forward(tokens=[t[i]]).cpu().numpy().copy())
    eng.cache.close_slot(s)
    check(np.concatenate(rows, 0), plain("A16", t), "bfloat16")


def test_sixteen_bit_kernels_against_the_plain_ones():
    """The bfloat16 path with the tensor-core kernels of the latent attention switched off gives the same logits within
    rounding: both are checked against the plain implementation above; here against each other, prompt and decoded."""
    from ghost_infer_b200.kernels import ops
    t = toks("C", 180, 77)
    outs = []
    for on in (True, False):
        old = dict(ops.TUNE)
        ops.TUNE["attn_latent_tc"] = ops.TUNE["bmm_heads_tc"] = on
        try:
            eng = engine_for("C", "bfloat16")
            s = eng.cache.open_slot()
            rows = [eng.step([gi.StepEntry(s, t[:170], list(range(170)))]).cpu().numpy()]
            run = eng.decoder([s], use_graph=False)
            rows += [run.forward(tokens=[x]).cpu().numpy().copy() for x in t[170:]]
            eng.cache.close_slot(s)
            outs.append(np.concatenate(rows, 0))
        finally:
            ops.TUNE.update(old)
    check(outs[0], outs[1], "bfloat16")


# ---- generation through the entry point ----------------------------------------------------------------------------------
def test_greedy_generation_through_the_entry_point(tmp_path):
    cfg, w, _ = made("A")
    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    pn.write_bf16_file(str(d / "model.safetensors"), w)
    llm = gi.LLM(str(d), dtype="float32", max_tokens=64 * 16, max_seq_len=512, beyond_trained_positions=True)
    prompts = [toks("A", n, 80 + i) for i, n in enumerate([3, 30, 11])]
    res = llm.generate(prompts, max_new=6, temperature=0.0, stop_token_ids=(), batch_size=2, max_step_tokens=16)
    for p, r in zip(prompts, res):
        seq = list(p)
        for _ in range(6):
            logits = pn.forward(cfg, w, seq)[-1]
            order = np.argsort(-logits, kind="stable")
            if logits[order[0]] - logits[order[1]] < 1e-3:
                break
            seq.append(int(order[0]))
        want = seq[len(p):]
        assert r.tokens[:len(want)] == want, f"prompt of {len(p)}: {r.tokens} vs {want}"
    assert llm.cache.free_pages == llm.cache.n_pages


# ---- configurations drawn at random ------------------------------------------------------------------------------------
def random_config(seed, all_experts, eights):
    r = np.random.default_rng(seed)
    pick = lambda xs: int(xs[r.integers(len(xs))])
    width = pick([40, 56, 72, 100, 132])

    def one_mixer():
        rot_dim = pick([8, 16, 24] if eights else [2, 6, 8, 12])
        return mixer(pick([1, 2, 3, 6, 17]), pick([4, 12, 16, 24]), rot_dim, pick([4, 8, 20]), pick([8, 24, 40, 72] if eights else [5, 18, 33]),
                     pick([8, 20, 36]), float(r.uniform(0.1, 0.5)), rot_dims=pick([rot_dim, max(2, rot_dim // 2 // 2 * 2)]),
                     base=float(10 ** r.uniform(1.5, 6)), scaling=pick([0, 1]) and (float(pick([1, 2, 8, 40])), pick([16, 64, 1024]), float(pick([4, 32])), float(pick([1, 2]))))

    def one_mlp():
        kind = pick([0, 1, 2])
        if kind == 0:
            return None
        if kind == 1:
            return dense(pick([24, 52, 64]))
        experts = pick([2, 5, 9])
        return moe(experts, experts if all_experts else pick([1, 2]), pick([8, 12, 40]))

    layers = []
    for i in range(pick([2, 3, 5])):
        if layers and r.random() < 0.4:
            j = pick(list(range(len(layers))))
            layers.append(layer(layers[j]["mixer"], layers[j]["mlp"], weights_of=j))
        else:
            layers.append(layer(one_mixer(), one_mlp()))
    return model_cfg(width, pick([50, 97, 260]), layers, eps=float(10 ** r.uniform(-6, -4)))


@pytest.mark.parametrize("seed,dtype", [(s, "float32") for s in range(6)] + [(s, "bfloat16") for s in range(100, 105)])
def test_configurations_drawn_at_random(seed, dtype):
    """Whole prompt, prompt cut in three, the tail token by token, and a batch of three, on a model nobody chose."""
    cfg = random_config(seed, all_experts=dtype == "bfloat16", eights=seed % 2 == 0)
    w = pn.random_weights(cfg, seed=seed)
    tensors = {k: torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16) for k, v in w.items()}
    model = gi.Model.from_config_dict(cfg).bind(tensors, dtype, "cuda:0")
    eng = gi.Engine(model, model.new_cache(max_tokens=64 * 24, max_seq_len=1024, beyond_trained_positions=True))
    r = np.random.default_rng(seed + 1)
    prompts = [r.integers(0, cfg["vocab"], size=n).tolist() for n in (150, 70, 9)]
    refs = [pn.forward(cfg, w, p) for p in prompts]
    check(run_whole(eng, prompts[0]), refs[0], dtype, f"{cfg}: whole")
    s = eng.cache.open_slot()
    rows = [eng.step([gi.StepEntry(s, prompts[0][a:b], list(range(b - a)))]).cpu().numpy() for a, b in ((0, 2), (2, 67), (67, 130))]
    run = eng.decoder([s])
    rows += [run.forward(tokens=[t]).cpu().numpy().copy() for t in prompts[0][130:]]
    eng.cache.close_slot(s)
    check(np.concatenate(rows, 0), refs[0], dtype, f"{cfg}: cut and decoded")
    slots = [eng.cache.open_slot() for _ in prompts]
    cut = [len(p) - 5 for p in prompts]
    out = eng.step([gi.StepEntry(sl, p[:c], list(range(c))) for sl, p, c in zip(slots, prompts, cut)]).cpu().numpy()
    got = [[out[sum(cut[:i]):sum(cut[:i + 1])]] for i in range(3)]
    run = eng.decoder(slots)
    for k in range(5):
        step_rows = run.forward(tokens=[p[c + k] for p, c in zip(prompts, cut)]).cpu().numpy()
        for i in range(3):
            got[i].append(step_rows[i:i + 1].copy())
    for sl in slots:
        eng.cache.close_slot(sl)
    for i in range(3):
        check(np.concatenate(got[i], 0), refs[i], dtype, f"{cfg}: request {i} of a batch")


# ---- the replay program as a user runs it ----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(tmp_path, dtype):
    """`bin/trace_run` on a model folder: requests whole, tails token by token, and unequal batches decoded together."""
    import subprocess
    import sys
    from test_gpu_trace_run import build_trace
    name = "B" if dtype == "float32" else "A16"
    cfg, w, _ = made(name)
    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    pn.write_bf16_file(str(d / "model.safetensors"), w)
    reqs, steps = build_trace({"vocab_size": cfg["vocab"]})
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(d), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", str(64 * 8)], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True,
                       text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-3000:]
    assert p.stdout.split("\n")[:len(steps)] == [f"done {i}" for i in range(len(steps))]
    refs = {rid: pn.forward(cfg, w, t) for rid, t in reqs.items()}
    place = {}
    for s in steps:
        want_rows = []
        for e in s["entries"]:
            base = place.get(e["id"], 0)
            want_rows += [refs[e["id"][:2]][base + k] for k in e["want"]]
            place[e["id"]] = base + len(e["tokens"])
        f = out / f"{s['step']}.f32"
        if want_rows:
            check(np.fromfile(f, dtype="<f4").reshape(-1, cfg["vocab"]), np.stack(want_rows), dtype, f"step {s['step']}")
        else:
            assert not f.exists()
