"""A plain, slow implementation of the Barovik decoder, used as the oracle of its tests.

Whole sequences, no cache, no batch, one function per mechanism, numpy only, float64 by default.  It shares no
code with the package under test.  Notation: T tokens, d the model's width; a matrix W is stored [out, in] and
applied to row vectors as h @ W.T.

The design: an embedding times a constant; layers of x += mixer(norm(x)), x += ff(norm(x)) (a layer may have no
feed-forward); the mixer is either attention inside chunks of positions with a capped score, a learned "sink" in
the softmax's denominator and values blended with those of the first blending layer, or a Mamba-2 state-space
layer; the feed-forward is either a gated dense one (tanh-form GELU) or a routed mixture of small SiLU-gated ones
with a shared one beside them; a final norm and an output matrix.
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np


# ---------------------------------------------------------------------------------------------------------------
# files
def read_safetensors(path, dtype=np.float64):
    """name -> array.  Layout: u64 header length, JSON header, raw little-endian data."""
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = data[b:e]
        dt = info["dtype"]
        if dt == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(dtype)
        elif dt == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(np.float32).astype(dtype)
        elif dt == "I32":
            arr = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"{name}: dtype {dt}")
        out[name] = arr.reshape(info["shape"])
    return out


def read_model(model_dir, dtype=np.float64):
    with open(f"{model_dir}/config.json") as f:
        cfg = json.load(f)
    return cfg, read_safetensors(f"{model_dir}/model.safetensors", dtype)


# ---------------------------------------------------------------------------------------------------------------
# small functions
def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def embed(table, tokens, scale):
    return table[np.asarray(tokens)] * scale


# ---------------------------------------------------------------------------------------------------------------
# the attention mixer
def visible(i, j, mask):
    """Whether the query at position i sees the key at position j."""
    if j > i:
        return False
    if mask and mask.get("size"):
        return i // int(mask["size"]) == j // int(mask["size"])
    return True


def sink_attention(h, w, m, v_first=None):
    """h [T, d] -> (output [T, d], the values this layer used [T, G * vdim]).

    m: the mixer's sizes and constants; w: its tensors by short name (q, k, v, o, sink, vmix).
    `v_first`: the values of the first blending layer for the same tokens, or None if this is that layer or the
    layer does not blend."""
    T = h.shape[0]
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w["q"].T).reshape(T, H, dk)
    k = (h @ w["k"].T).reshape(T, G, dk)
    v = h @ w["v"].T
    if v_first is not None:
        lam = float(w["vmix"])
        v = (1.0 - lam) * v + lam * v_first
    vh = v.reshape(T, G, dv)
    cap = m.get("softcap")
    out = np.zeros((T, H, dv), dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, m.get("mask"))]
            s = np.array([q[i, head] @ k[j, g] for j in js]) * float(m["scale"])
            if cap:
                s = float(cap) * np.tanh(s / float(cap))
            top = max(s.max(), float(w["sink"][head])) if "sink" in w else s.max()
            e = np.exp(s - top)
            denom = e.sum() + (math.exp(float(w["sink"][head]) - top) if "sink" in w else 0.0)
            out[i, head] = (e / denom) @ vh[js, g]
    return out.reshape(T, H * dv) @ w["o"].T, v


# ---------------------------------------------------------------------------------------------------------------
# the state-space mixer
def causal_conv(u, taps_w, bias):
    """u [T, C], taps_w [C, K] (its last column multiplies the current token), zeros before the start."""
    T, C = u.shape
    K = taps_w.shape[1]
    padded = np.concatenate([np.zeros((K - 1, C), dtype=u.dtype), u], axis=0)
    out = np.zeros_like(u)
    for t in range(T):
        out[t] = (padded[t:t + K].T * taps_w).sum(axis=1) + bias
    return out


def ssm_scan(x, B, C, dt, a_log, D, heads, groups):
    """x [T, heads, P], B and C [T, groups, N], dt [T, heads] (after softplus) -> y [T, heads, P].
    Per head: S <- exp(-exp(a_log) dt) S + dt B x^T (S is N x P), y = S^T C + D x."""
    T, _, P = x.shape
    N = B.shape[2]
    y = np.zeros_like(x)
    for hd in range(heads):
        g = hd // (heads // groups)
        S = np.zeros((N, P), dtype=x.dtype)
        for t in range(T):
            S = math.exp(-math.exp(float(a_log[hd])) * float(dt[t, hd])) * S + float(dt[t, hd]) * np.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + float(D[hd]) * x[t, hd]
    return y


def mamba2(h, w, m, eps):
    T = h.shape[0]
    heads, P, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = heads * P
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    assert dt.shape[1] == heads
    xbc = silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].reshape(T, heads, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w["dt_bias"])
    y = ssm_scan(x, B, C, dt, w["A_log"], w["D"], heads, G).reshape(T, inner)
    y = y * silu(z)
    parts = int(m["norm_groups"])
    y = rms_norm(y.reshape(T, parts, inner // parts), 1.0, eps).reshape(T, inner) * w["norm"]
    return y @ w["o"].T


# ---------------------------------------------------------------------------------------------------------------
# feed-forwards
def gated_ff(h, w, act):
    return (act(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def routed_ff(h, w, mlp):
    """w: tensors under the feed-forward's prefix (router, e<i>.gate/up/down, shared.*)."""
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    logits = h @ w["router"].T
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = np.argsort(-logits[t], kind="stable")[:top]
        e = np.exp(logits[t, chosen] - logits[t, chosen].max())
        weights = e / e.sum()
        for idx, wt in zip(chosen, weights):
            sub = {k: w[f"e{idx}.{k}"] for k in ("gate", "up", "down")}
            out[t] += wt * gated_ff(h[t:t + 1], sub, silu)[0]
    if mlp.get("shared"):
        sub = {k: w[f"shared.{k}"] for k in ("gate", "up", "down")}
        out = out + sigmoid(h @ w["shared.sg"].T) * gated_ff(h, sub, silu)
    return out


# ---------------------------------------------------------------------------------------------------------------
# the model
def under(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg, weights, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence.  `layers_out`: a list that receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = embed(weights["embed"], tokens, float(cfg["embedding"]["scale"]))
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        w = under(weights, f"l{i}.")
        h = rms_norm(x, w["norm1"], eps)
        m = layer["mixer"]
        if layer["type"] == "attention":
            blend = bool(m.get("v_mix"))
            y, v = sink_attention(h, under(w, "mix."), m, v_first if blend else None)
            if blend and v_first is None:
                v_first = v
        elif layer["type"] == "mamba2":
            y = mamba2(h, under(w, "mix."), m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + y
        mlp = layer.get("mlp")
        if mlp:
            h = rms_norm(x, w["norm2"], eps)
            if mlp["kind"] == "dense":
                x = x + gated_ff(h, under(w, "mlp."), gelu_tanh)
            elif mlp["kind"] == "moe":
                x = x + routed_ff(h, under(w, "mlp."), mlp)
            else:
                raise ValueError(mlp["kind"])
        if layers_out is not None:
            layers_out.append(x.copy())
    return rms_norm(x, weights["final.norm"], eps) @ weights["head"].T


# ---------------------------------------------------------------------------------------------------------------
# random models for tests
def random_weights(cfg, seed=0, dtype=np.float64):
    """Weights for `cfg`, rounded to bfloat16 values so that a bfloat16 file holds them exactly."""
    rng = np.random.default_rng(seed)
    d, out = int(cfg["width"]), {}

    def put(name, shape, std=None, mean=0.0):
        std = std if std is not None else 1.0 / math.sqrt(shape[-1]) if len(shape) > 1 else 0.5
        a = (rng.standard_normal(shape) * std + mean).astype(np.float32)
        u = a.view(np.uint32).astype(np.uint64)
        r = (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32)
        out[name] = r.view(np.float32).astype(dtype).reshape(shape)

    put("embed", (int(cfg["vocab"]), d), 1.0)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        put(p + "norm1", (d,), 0.1, 1.0)
        if layer["type"] == "attention":
            H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            put(p + "mix.q", (H * dk, d)); put(p + "mix.k", (G * dk, d)); put(p + "mix.v", (G * dv, d))
            put(p + "mix.sink", (H,), 1.0); put(p + "mix.o", (d, H * dv))
            if m.get("v_mix"):
                put(p + "mix.vmix", (), 0.2, 0.4)
        else:
            heads, P, N, G, K = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"]), int(m["conv"])
            inner, ch = heads * P, heads * P + 2 * G * N
            put(p + "mix.in", (2 * inner + 2 * G * N + heads, d)); put(p + "mix.conv", (ch, K), 0.5)
            put(p + "mix.conv.b", (ch,), 0.2); put(p + "mix.dt_bias", (heads,), 0.5, -1.0)
            put(p + "mix.A_log", (heads,), 0.5, -0.5); put(p + "mix.D", (heads,), 0.5, 1.0)
            put(p + "mix.norm", (inner,), 0.1, 1.0); put(p + "mix.o", (d, inner))
        mlp = layer.get("mlp")
        if not mlp:
            continue
        put(p + "norm2", (d,), 0.1, 1.0)
        if mlp["kind"] == "dense":
            f = int(mlp["ff"])
            put(p + "mlp.gate", (f, d)); put(p + "mlp.up", (f, d)); put(p + "mlp.down", (d, f))
        else:
            f = int(mlp["expert"]["ff"])
            for e in range(int(mlp["router"]["experts"])):
                put(p + f"mlp.e{e}.gate", (f, d)); put(p + f"mlp.e{e}.up", (f, d)); put(p + f"mlp.e{e}.down", (d, f))
            put(p + "mlp.router", (int(mlp["router"]["experts"]), d), 4.0 / math.sqrt(d))
            if mlp.get("shared"):
                f = int(mlp["shared"]["ff"])
                put(p + "mlp.shared.gate", (f, d)); put(p + "mlp.shared.up", (f, d)); put(p + "mlp.shared.down", (d, f))
                put(p + "mlp.shared.sg", (1, d))
    put("final.norm", (d,), 0.1, 1.0)
    put("head", (int(cfg["vocab"]), d))
    return out


def write_safetensors_bf16(path, tensors):
    """Writes float arrays as bfloat16 (the values must be bfloat16 values already) in the safetensors layout."""
    header, blobs, at = {}, [], 0
    for name, a in tensors.items():
        raw = (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype("<u2").tobytes()
        header[name] = {"dtype": "BF16", "shape": list(a.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for b in blobs:
            f.write(b)
