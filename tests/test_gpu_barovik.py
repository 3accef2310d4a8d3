"""The Barovik decoder through the engine, against the plain implementation (`plain_barovik.py`).

Every test makes its own small configuration and random weights.  The configurations differ from each other in every
size and constant and exercise the values that are easily 1 or equal: one kv head and as many kv heads as heads, one
group and several, one norm group and several, values wider and narrower than keys, a chunk of 7 positions (an edge
every few tokens) and one of 130 (across two page borders), two to four convolution taps, one expert chosen and all of
them, with and without a shared expert, a layer without feed-forward, a model that starts with a state-space layer,
layers that blend values and one that does not.  Scores are made sharp (queries and keys scaled up) so that one key
more or less at a chunk's edge, or a sink left out, moves the logits by far more than the tolerance.
"""
import json
import os

import numpy as np
import pytest
import torch

import ghost_infer_b200 as gi
import plain_barovik as pb

pytestmark = pytest.mark.gpu


def attn(heads, kv, dim, vdim, chunk, scale, cap=None, v_mix=True):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if chunk:
        m["mask"] = {"size": chunk}
    if cap:
        m["softcap"] = cap
    return m


def ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def model_cfg(width, vocab, layers, scale=0.7, eps=1e-5):
    return {"architecture": "Barovik", "width": width, "vocab": vocab, "embedding": {"scale": scale}, "norm": {"eps": eps},
            "layers": layers}


CFG_A = model_cfg(96, 200, [
    layer("attention", attn(4, 2, 32, 16, 24, 0.5, cap=20.0), dense(136)),
    layer("mamba2", ssm(4, 16, 16, 2, 3, 2), moe(6, 2, 40, shared=56)),
    layer("attention", attn(4, 2, 32, 16, 24, 0.5, cap=20.0), moe(5, 1, 24)),
    layer("mamba2", ssm(3, 24, 8, 1, 4, 1), None),
    layer("attention", attn(3, 3, 16, 40, 130, 0.6, v_mix=False), dense(64)),
])
CFG_B = model_cfg(80, 301, [
    layer("mamba2", ssm(2, 24, 24, 2, 2, 3), dense(72)),
    layer("attention", attn(5, 1, 48, 80, 7, 0.3, cap=8.0), moe(3, 3, 32, shared=16)),
    layer("attention", attn(5, 1, 48, 80, 7, 0.3), None),
], scale=1.3, eps=3e-6)
# For the bfloat16 path: a router that sees activations rounded to 8 bits picks, on a near tie, another expert than the
# oracle (with random weights a few tokens in a hundred have two candidates within the rounding), and a state-space layer
# behind it remembers the difference for the rest of the sequence.  Where every expert is chosen (top = experts) the
# output is a continuous function of the logits, so these models can be compared row by row in 16 bits; routing to a few
# of many is pinned in 32 bits, and in 16 bits on the same inputs by `test_routed_experts_in_bfloat16`.
CFG_A16 = json.loads(json.dumps(CFG_A))
for _l in CFG_A16["layers"]:
    if _l["mlp"] and _l["mlp"]["kind"] == "moe":
        _l["mlp"]["router"]["top"] = _l["mlp"]["router"]["experts"]
# Keys and values of 64 values each: the sizes for which prompts run on the tcgen05 attention kernel in 16 bits.
CFG_C = model_cfg(128, 150, [
    layer("attention", attn(4, 2, 64, 64, 50, 0.2, cap=15.0), dense(96)),
    layer("mamba2", ssm(2, 32, 16, 1, 4, 1), moe(4, 4, 32, shared=32)),
    layer("attention", attn(4, 2, 64, 64, 50, 0.2, cap=15.0), None),
])
CONFIGS = {"A": CFG_A, "A16": CFG_A16, "B": CFG_B, "C": CFG_C}
_made = {}


def made(name):
    """(configuration, float64 weights of bfloat16 values, torch tensors for binding)."""
    if name not in _made:
        cfg = CONFIGS[name]
        w = pb.random_weights(cfg, seed=len(name) + ord(name[0]))
        # sharp scores: an edge or a sink that is off shows in the logits (not for the model that is only run in 16
        # bits: sharp scores also multiply what the rounding of queries and keys does to the softmax)
        for k in w:
            if name not in ("A16", "C") and (k.endswith("mix.q") or k.endswith("mix.k")):
                w[k] = w[k] * 2.0
        _made[name] = (cfg, w, {k: torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16) for k, v in w.items()})
    return _made[name]


def engine_for(name, dtype, max_tokens=64 * 40, max_slots=None):
    cfg, _, tensors = made(name)
    model = gi.Model.from_config_dict(cfg).bind(tensors, dtype, "cuda:0")
    cache = model.new_cache(max_tokens=max_tokens, max_seq_len=4096, max_slots=max_slots)
    return gi.Engine(model, cache)


_plain = {}


def plain(name, tokens):
    key = (name, tuple(tokens))
    if key not in _plain:
        cfg, w, _ = made(name)
        _plain[key] = pb.forward(cfg, w, list(tokens))
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


# ---- each mechanism alone: one-layer models ------------------------------------------------------------------------
ALONE = {
    "attention": layer("attention", attn(4, 2, 16, 24, 10, 0.4, cap=5.0, v_mix=False), None),
    "attention_plain": layer("attention", attn(2, 2, 24, 24, None, 0.3, v_mix=False), None),
    "mamba2": layer("mamba2", ssm(4, 8, 12, 2, 4, 2), None),
    "dense": layer("mamba2", ssm(1, 8, 4, 1, 1, 1), dense(52)),
    "moe": layer("mamba2", ssm(1, 8, 4, 1, 2, 1), moe(7, 3, 20, shared=12)),
}


@pytest.mark.parametrize("which", sorted(ALONE))
def test_each_mechanism_alone(which):
    cfg = model_cfg(48, 90, [ALONE[which]], scale=1.0)
    w = pb.random_weights(cfg, seed=11)
    tensors = {k: torch.from_numpy(np.asarray(v, dtype=np.float32)) for k, v in w.items()}
    model = gi.Model.from_config_dict(cfg).bind(tensors, "float32", "cuda:0")
    eng = gi.Engine(model, model.new_cache(max_tokens=256, max_seq_len=256))
    tokens = np.random.default_rng(5).integers(0, 90, size=45).tolist()
    check(run_whole(eng, tokens), pb.forward(cfg, w, tokens), "float32", which)


def test_value_blending_uses_the_first_blending_layer():
    """Three blending layers: the third must blend with the first one's values, not the second's."""
    a = attn(2, 1, 16, 8, 9, 0.5, v_mix=True)
    cfg = model_cfg(32, 60, [layer("attention", a, None), layer("attention", a, None), layer("attention", a, None)])
    w = pb.random_weights(cfg, seed=3)
    tensors = {k: torch.from_numpy(np.asarray(v, dtype=np.float32)) for k, v in w.items()}
    model = gi.Model.from_config_dict(cfg).bind(tensors, "float32", "cuda:0")
    eng = gi.Engine(model, model.new_cache(max_tokens=128, max_seq_len=128))
    tokens = np.random.default_rng(1).integers(0, 60, size=30).tolist()
    check(run_whole(eng, tokens), pb.forward(cfg, w, tokens), "float32")


def test_routed_experts_in_bfloat16():
    """A few of many experts in 16 bits, on the same inputs as in 32 bits (the router then makes the same choices): the
    sort by expert, the experts' products over their own rows and the weighted sum back into the stream."""
    from ghost_infer_b200.kernels import ops
    g = torch.Generator().manual_seed(4)
    T, d, E, top, f = 150, 64, 9, 2, 24
    h = torch.randn(T, d, generator=g).to(torch.bfloat16)
    wr = (torch.randn(E, d, generator=g) * 0.3).to(torch.bfloat16)
    wgu = (torch.randn(E, 2 * f, d, generator=g) * 0.15).to(torch.bfloat16)
    wd = (torch.randn(E, d, f, generator=g) * 0.2).to(torch.bfloat16)
    outs = {}
    for dt in (torch.float32, torch.bfloat16):
        hh, r, gu, dn = (t.to("cuda", dt).contiguous() for t in (h, wr, wgu, wd))
        ids, wts, _ = ops.moe_route(hh, r, top)
        offsets, perm, inv = ops.moe_plan(ids, E)
        down = ops.moe_experts(hh, gu, dn, offsets, perm, top)
        x = torch.zeros(T, d, device="cuda")
        ops.moe_combine(x, down, inv, wts)
        outs[dt] = (ids.cpu(), offsets.cpu(), x.cpu())
    assert torch.equal(outs[torch.float32][0], outs[torch.bfloat16][0]) and torch.equal(outs[torch.float32][1], outs[torch.bfloat16][1])
    ids, offsets, x32 = outs[torch.float32]
    assert offsets.tolist() == np.concatenate([[0], np.cumsum(np.bincount(ids.reshape(-1).numpy(), minlength=E))]).tolist()
    hd, logits = h.double(), h.double() @ wr.double().T
    want = torch.zeros(T, d, dtype=torch.float64)
    for t in range(T):
        chosen = ids[t].long()
        p = torch.softmax(logits[t, chosen], 0)
        for e, pe in zip(chosen.tolist(), p):
            gate, up = wgu[e, :f].double() @ hd[t], wgu[e, f:].double() @ hd[t]
            want[t] += pe * (wd[e].double() @ (torch.nn.functional.silu(gate) * up))
    assert (x32.double() - want).abs().max() < 1e-4
    assert (outs[torch.bfloat16][2].double() - want).abs().max() < 0.03 * float(want.abs().max())


# ---- whole prompts, tails token by token, portions -----------------------------------------------------------------
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A16", "bfloat16"), ("B", "float32"), ("B", "bfloat16"), ("C", "bfloat16"),
                                        ("C", "float32")])
def test_whole_prompt(name, dtype):
    eng = engine_for(name, dtype)
    for n, seed in ((1, 1), (2, 2), (150, 3)):       # the first tokens of a sequence, and chunk and page borders
        t = toks(name, n, seed)
        check(run_whole(eng, t), plain(name, t), dtype, f"{n} tokens")


@pytest.mark.parametrize("name,dtype,graph", [("A", "float32", True), ("A16", "bfloat16", True), ("B", "float32", False),
                                              ("B", "float32", True), ("C", "bfloat16", True)])
def test_prompt_then_token_by_token(name, dtype, graph):
    """Decoding crosses chunk edges (every 7 or 24 positions), a page border (64, 128) and the state's every step."""
    eng = engine_for(name, dtype)
    t = toks(name, 140, 7)
    ref = plain(name, t)
    s = eng.cache.open_slot()
    cut = 50
    rows = [eng.step([gi.StepEntry(s, t[:cut], list(range(cut)))]).cpu().numpy()]
    run = eng.decoder([s], use_graph=graph)
    for i in range(cut, len(t)):
        rows.append(run.forward(tokens=[t[i]]).cpu().numpy().copy())
    eng.cache.close_slot(s)
    check(np.concatenate(rows, 0), ref, dtype)


def test_decoding_from_the_first_token():
    eng = engine_for("B", "float32")
    t = toks("B", 40, 9)
    s = eng.cache.open_slot()
    rows = [eng.step([gi.StepEntry(s, t[i:i + 1], [0])]).cpu().numpy() for i in range(len(t))]
    eng.cache.close_slot(s)
    check(np.concatenate(rows, 0), plain("B", t), "float32")


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("A16", "bfloat16"), ("C", "bfloat16")])
def test_portions_of_several_sizes(name, dtype):
    eng = engine_for(name, dtype)
    t = toks(name, 200, 13)
    ref = plain(name, t)
    for sizes in ([2, 2, 3, 17, 64, 2, 65, 45], [31, 1, 1, 2, 100, 65], [7] * 28 + [4]):
        assert sum(sizes) == len(t)
        s = eng.cache.open_slot()
        rows, at = [], 0
        for n in sizes:
            rows.append(eng.step([gi.StepEntry(s, t[at:at + n], list(range(n)))]).cpu().numpy())
            at += n
        eng.cache.close_slot(s)
        check(np.concatenate(rows, 0), ref, dtype, f"portions {sizes[:4]}...")


def test_float32_does_not_depend_on_the_cut():
    """The 32-bit recurrence and products take the same order however a prompt is cut: the state-space layers give the
    same bits; attention differs between its prompt and its one-token kernel by rounding only."""
    cfg = model_cfg(48, 90, [ALONE["mamba2"], ALONE["moe"]])
    w = pb.random_weights(cfg, seed=2)
    tensors = {k: torch.from_numpy(np.asarray(v, dtype=np.float32)) for k, v in w.items()}
    model = gi.Model.from_config_dict(cfg).bind(tensors, "float32", "cuda:0")
    eng = gi.Engine(model, model.new_cache(max_tokens=512, max_seq_len=256))
    t = np.random.default_rng(4).integers(0, 90, size=70).tolist()
    whole = run_whole(eng, t)
    s = eng.cache.open_slot()
    rows, at = [], 0
    for n in [3, 16, 1, 17, 33]:
        rows.append(eng.step([gi.StepEntry(s, t[at:at + n], list(range(n)))]).cpu().numpy())
        at += n
    eng.cache.close_slot(s)
    assert np.array_equal(np.concatenate(rows, 0), whole)


# ---- batches -----------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("A16", "bfloat16")])
def test_unequal_batch_against_each_alone(name, dtype):
    eng = engine_for(name, dtype)
    lens = [1, 66, 23, 131]
    prompts = [toks(name, n + 12, 20 + i) for i, n in enumerate(lens)]
    slots = [eng.cache.open_slot() for _ in prompts]
    out = eng.step([gi.StepEntry(s, p[:n], list(range(n))) for s, p, n in zip(slots, prompts, lens)]).cpu().numpy()
    got = [[out[sum(lens[:i]):sum(lens[:i + 1])]] for i in range(len(lens))]
    live = list(range(len(prompts)))
    for step in range(12):                       # decoded together; the shortest leaves half way
        if step == 6:
            eng.cache.close_slot(slots[0])
            live = live[1:]
        run = eng.decoder([slots[i] for i in live])
        rows = run.forward(tokens=[prompts[i][lens[i] + step] for i in live]).cpu().numpy()
        for j, i in enumerate(live):
            got[i].append(rows[j:j + 1].copy())
    for i in live:
        eng.cache.close_slot(slots[i])
    for i, p in enumerate(prompts):
        g = np.concatenate(got[i], 0)
        check(g, plain(name, p)[:len(g)], dtype, f"request {i}")
    assert eng.cache.free_pages == eng.cache.n_pages


def test_mixed_step_of_fresh_prompts_and_sequences_under_way():
    eng = engine_for("A", "float32")
    a, b = toks("A", 90, 31), toks("A", 40, 32)
    sa, sb = eng.cache.open_slot(), eng.cache.open_slot()
    r0 = eng.step([gi.StepEntry(sa, a[:50], list(range(50)))]).cpu().numpy()
    r1 = eng.step([gi.StepEntry(sb, b, list(range(40))), gi.StepEntry(sa, a[50:51], [0])]).cpu().numpy()
    r2 = eng.step([gi.StepEntry(sa, a[51:], list(range(39)))]).cpu().numpy()
    check(np.concatenate([r0, r1[40:], r2], 0), plain("A", a), "float32", "under way")
    check(r1[:40], plain("A", b), "float32", "fresh")


# ---- pages and slots given back and used again ---------------------------------------------------------------------
def test_slots_and_pages_used_again():
    """A pool of five pages and two slots: sequences come and go; whoever gets a used slot must find its state zero and
    must not see the keys the pages held before."""
    eng = engine_for("A", "float32", max_tokens=64 * 5, max_slots=2)
    for round_ in range(3):
        p, q = toks("A", 100 + round_, 40 + round_), toks("A", 70, 50 + round_)
        s1, s2 = eng.cache.open_slot(), eng.cache.open_slot()
        out = eng.step([gi.StepEntry(s1, p, [len(p) - 1]), gi.StepEntry(s2, q, list(range(70)))]).cpu().numpy()
        check(out[0], plain("A", p)[-1], "float32", f"round {round_}")
        check(out[1:], plain("A", q), "float32", f"round {round_}")
        eng.cache.close_slot(s1)
        eng.cache.close_slot(s2)
    assert eng.cache.free_pages == eng.cache.n_pages


def test_a_chunked_cache_gives_pages_back_as_it_goes():
    """Chunks of 7 positions: a sequence of 700 tokens lives in a pool of three pages, because pages wholly before the
    newest token's chunk are given back."""
    eng = engine_for("B", "float32", max_tokens=64 * 3, max_slots=1)
    t = toks("B", 700, 61)
    s = eng.cache.open_slot()
    rows, at = [], 0
    while at < len(t):
        n = min(50, len(t) - at)
        rows.append(eng.step([gi.StepEntry(s, t[at:at + n], list(range(n)))]).cpu().numpy())
        at += n
    assert eng.cache.free_pages >= 1
    eng.cache.close_slot(s)
    check(np.concatenate(rows, 0), plain("B", t), "float32")


# ---- edges made to show ------------------------------------------------------------------------------------------------
def test_the_key_outside_the_chunk_is_not_seen_and_the_one_inside_is():
    """One attention layer whose token 5 is a key every query loves (score far above the rest) and whose value is
    unlike the others: queries of its chunk follow it, the first query of the next chunk must not."""
    chunk = 12
    cfg = model_cfg(32, 16, [layer("attention", attn(2, 1, 16, 16, chunk, 1.0, v_mix=False), None)], scale=1.0)
    w = pb.random_weights(cfg, seed=8)
    w["embed"][:] = 0.0
    w["embed"][:, :8] = np.random.default_rng(0).standard_normal((16, 8)).round(1) * 0.25
    w["embed"][5] = 0.0
    w["embed"][5, 8] = 4.0                                  # the loved token has a direction of its own
    w["embed"][:, 9] = 1.0                                  # and every token one they all share
    w["l0.norm1"][:] = 1.0
    w["l0.mix.q"][:] = 0.0
    w["l0.mix.k"][:] = 0.0
    w["l0.mix.q"][[0, 16], 9] = 1.0                         # every query is the shared direction ...
    w["l0.mix.k"][0, 8] = 8.0                               # ... and only token 5 has a key for it
    w["l0.mix.sink"][:] = -4.0
    tensors = {k: torch.from_numpy(np.asarray(v, dtype=np.float32)) for k, v in w.items()}
    model = gi.Model.from_config_dict(cfg).bind(tensors, "float32", "cuda:0")
    eng = gi.Engine(model, model.new_cache(max_tokens=256, max_seq_len=256))
    rng = np.random.default_rng(6)
    t = [int(x) for x in rng.integers(6, 16, size=40)]
    t[chunk - 2] = 5                                        # position 10: seen by 10 and 11, not by 12
    t[2 * chunk] = 5                                        # position 24, the first of its chunk: seen by 24..35
    ref = pb.forward(cfg, w, t)
    assert np.abs(ref[chunk - 1] - ref[chunk]).max() > 0.1   # the edge is visible in the oracle itself
    check(run_whole(eng, t), ref, "float32", "whole")
    s = eng.cache.open_slot()
    rows = [eng.step([gi.StepEntry(s, t[:chunk - 1], list(range(chunk - 1)))]).cpu().numpy()]
    run = eng.decoder([s])
    for i in range(chunk - 1, len(t)):
        rows.append(run.forward(tokens=[t[i]]).cpu().numpy().copy())
    eng.cache.close_slot(s)
    check(np.concatenate(rows, 0), ref, "float32", "decoded")


def test_a_sink_left_out_would_show():
    cfg = model_cfg(32, 40, [layer("attention", attn(2, 2, 8, 8, 9, 0.5, v_mix=False), None)])
    w = pb.random_weights(cfg, seed=9)
    w["l0.mix.sink"][:] = [3.0, -1.0]
    tensors = {k: torch.from_numpy(np.asarray(v, dtype=np.float32)) for k, v in w.items()}
    model = gi.Model.from_config_dict(cfg).bind(tensors, "float32", "cuda:0")
    eng = gi.Engine(model, model.new_cache(max_tokens=128, max_seq_len=128))
    t = np.random.default_rng(2).integers(0, 40, size=30).tolist()
    ref = pb.forward(cfg, w, t)
    w2 = dict(w)
    w2["l0.mix.sink"] = np.full(2, -60.0)
    assert np.abs(pb.forward(cfg, w2, t) - ref).max() > 0.05
    check(run_whole(eng, t), ref, "float32")


# ---- long decoding -------------------------------------------------------------------------------------------------
def test_long_decoding_through_the_graph_runner():
    """320 decoded tokens: the 256-position length bucket, five page borders, dozens of chunk edges."""
    eng = engine_for("A16", "bfloat16")
    t = toks("A16", 330, 71)
    s = eng.cache.open_slot()
    rows = [eng.step([gi.StepEntry(s, t[:10], list(range(10)))]).cpu().numpy()]
    run = eng.decoder([s])
    for i in range(10, len(t)):
        rows.append(run.forward(tokens=[t[i]]).cpu().numpy().copy())
    eng.cache.close_slot(s)
    check(np.concatenate(rows, 0), plain("A16", t), "bfloat16")


# ---- generation through the entry point ----------------------------------------------------------------------------------
def test_greedy_generation_through_the_entry_point(tmp_path):
    cfg, w, _ = made("A")
    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    pb.write_safetensors_bf16(str(d / "model.safetensors"), w)
    llm = gi.LLM(str(d), dtype="float32", max_tokens=64 * 16, max_seq_len=512)
    prompts = [toks("A", n, 80 + i) for i, n in enumerate([3, 30, 11])]
    res = llm.generate(prompts, max_new=6, temperature=0.0, stop_token_ids=(), batch_size=2, max_step_tokens=16)
    for p, r in zip(prompts, res):
        seq = list(p)
        for _ in range(6):
            logits = pb.forward(cfg, w, seq)[-1]
            order = np.argsort(-logits, kind="stable")
            if logits[order[0]] - logits[order[1]] < 1e-3:
                break
            seq.append(int(order[0]))
        want = seq[len(p):]
        assert r.tokens[:len(want)] == want, f"prompt of {len(p)}: {r.tokens} vs {want}"
    assert llm.cache.free_pages == llm.cache.n_pages


# ---- configurations drawn at random ------------------------------------------------------------------------------------
def random_config(seed, all_experts):
    """Sizes drawn from lists that mix multiples of 8 with numbers that are not (which take the kernels' plain paths)."""
    r = np.random.default_rng(seed)
    pick = lambda xs: int(xs[r.integers(len(xs))])
    width = pick([40, 56, 72, 100, 132])
    kv, vdim_att = pick([1, 2, 3]), pick([8, 12, 24, 40])
    shared_attention = attn(kv * pick([1, 2, 4]), kv, pick([8, 20, 32, 48]), vdim_att, pick([5, 17, 64, 90]),
                            float(r.uniform(0.1, 0.5)), cap=pick([0, 7, 40]) or None, v_mix=True)
    layers = []
    for _ in range(pick([2, 3, 4])):
        if r.random() < 0.5:
            mixer = ("attention", shared_attention if r.random() < 0.7 else
                     attn(pick([2, 4]), pick([1, 2]), pick([16, 24]), pick([16, 10]), pick([9, 33]), 0.3, v_mix=False))
        else:
            groups = pick([1, 2])
            mixer = ("mamba2", ssm(groups * pick([1, 2, 3]), pick([4, 10, 16, 36]), pick([3, 16, 40, 130]), groups, pick([1, 2, 4, 5]), 1))
            if (mixer[1]["heads"] * mixer[1]["vdim"]) % 2 == 0 and r.random() < 0.5:
                mixer[1]["norm_groups"] = 2
        kind = pick([0, 1, 2])
        if kind == 0:
            mlp = None
        elif kind == 1:
            mlp = dense(pick([24, 52, 64]))
        else:
            experts = pick([2, 5, 9])
            mlp = moe(experts, experts if all_experts else pick([1, 2]), pick([8, 12, 40]), shared=pick([0, 16, 20]) or None)
        layers.append(layer(mixer[0], mixer[1], mlp))
    return model_cfg(width, pick([50, 97, 260]), layers, scale=float(r.uniform(0.5, 2.0)), eps=float(10 ** r.uniform(-6, -4)))


@pytest.mark.parametrize("seed,dtype", [(s, "float32") for s in range(6)] + [(s, "bfloat16") for s in range(100, 104)])
def test_configurations_drawn_at_random(seed, dtype):
    """Whole prompt, prompt cut in three, the tail token by token, and a batch of three, on a model nobody chose."""
    cfg = random_config(seed, all_experts=dtype == "bfloat16")
    w = pb.random_weights(cfg, seed=seed)
    tensors = {k: torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16) for k, v in w.items()}
    model = gi.Model.from_config_dict(cfg).bind(tensors, dtype, "cuda:0")
    eng = gi.Engine(model, model.new_cache(max_tokens=64 * 24, max_seq_len=1024))
    r = np.random.default_rng(seed + 1)
    prompts = [r.integers(0, cfg["vocab"], size=n).tolist() for n in (150, 70, 9)]
    refs = [pb.forward(cfg, w, p) for p in prompts]
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
    cfg, w, _ = made("B")
    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    pb.write_safetensors_bf16(str(d / "model.safetensors"), w)
    reqs, steps = build_trace({"vocab_size": cfg["vocab"]})
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(d), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", str(64 * 8)], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True,
                       text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-3000:]
    assert p.stdout.split("\n")[:len(steps)] == [f"done {i}" for i in range(len(steps))]
    refs = {rid: pb.forward(cfg, w, toks) for rid, toks in reqs.items()}
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
