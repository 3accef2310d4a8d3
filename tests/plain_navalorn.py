"""A plain, slow implementation of the Navalorn decoder in numpy float64: one function per mechanism.

It shares no code with the package.  Everything is recomputed for the whole sequence at every call (no cache), and
the attention is written in its direct form: every head gets its own keys and values out of the latent.

Notation: T tokens, width d, H heads; a head's query and key are [dn unrotated | dr rotated] numbers, its value dv
numbers; the keys' and values' latent has r numbers, the queries' latent rq.
"""
from __future__ import annotations

import math

import numpy as np


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis; var is the mean squared deviation; no bias."""
    x = np.asarray(x, dtype=np.float64)
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * np.asarray(w, dtype=np.float64)


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * np.asarray(w, dtype=np.float64)


def rotary_frequencies(dims, base, scaling):
    """(frequency per pair [dims / 2], factor on cos and sin).  Pair i turns by position * f_i, f_i = base^(-2i / dims).
    With `scaling` (factor, original, fast, slow) the frequencies are stretched YaRN-wise: pairs that turn often within
    the original length keep f_i, those that turn rarely get f_i / factor, with a linear ramp over the pair index
    between the indices where a pair makes `fast` and `slow` turns over `original` positions."""
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)], dtype=np.float64)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((np.arange(half, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, freqs, magnitude):
    """x [T, ..., dims]: numbers 2i and 2i + 1 are a pair (u, v) -> (u c - v s, v c + u s), c and s the cosine and sine
    of position * freqs[i], both times `magnitude`."""
    x = np.asarray(x, dtype=np.float64)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freqs[None, :]          # [T, dims / 2]
    c, s = np.cos(ang) * magnitude, np.sin(ang) * magnitude
    while c.ndim < x.ndim:
        c, s = c[:, None], s[:, None]
    u, v = x[..., 0::2], x[..., 1::2]
    out = np.empty_like(x)
    out[..., 0::2] = u * c - v * s
    out[..., 1::2] = v * c + u * s
    return out


def latent_attention(h, w, m, eps, positions=None):
    """The mixer over a whole sequence.  `w`: the mixer's tensors by short name (dq, dq.norm, uq, dkv, dkv.norm, uk, uv,
    o); `m`: its sizes and constants (heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot)."""
    h = np.asarray(h, dtype=np.float64)
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T) if positions is None else np.asarray(positions)
    f64 = lambda name: np.asarray(w[name], dtype=np.float64)
    cq = rms_norm(h @ f64("dq").T, w["dq.norm"], eps)
    q = (cq @ f64("uq").T).reshape(T, H, dn + dr)
    down = h @ f64("dkv").T
    c = rms_norm(down[:, :r], w["dkv.norm"], eps)
    k_rot = down[:, r:]                                                       # [T, dr], one for all heads
    q_rot, k_rot = q[:, :, dn:].copy(), k_rot.copy()
    if dr:
        rot = m["rot"]
        freqs, mag = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        nrot = rot["dims"]
        q_rot[..., :nrot] = rotate_pairs(q_rot[..., :nrot], pos, freqs, mag)
        k_rot[:, :nrot] = rotate_pairs(k_rot[:, :nrot], pos, freqs, mag)
    k = (c @ f64("uk").T).reshape(T, H, dn)
    v = (c @ f64("uv").T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for hd in range(H):
        s = (q[:, hd, :dn] @ k[:, hd, :].T + q_rot[:, hd, :] @ k_rot.T) * m["scale"]      # [T, T]
        s = np.where(pos[None, :] <= pos[:, None], s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(axis=-1, keepdims=True)
        out[:, hd, :] = p @ v[:, hd, :]
    return out.reshape(T, H * dv) @ f64("o").T


def relu_squared(z):
    return np.maximum(z, 0.0) ** 2


def dense_feed_forward(h, w):
    """W_down relu(W_up h + b_up)^2 + b_down."""
    f64 = lambda name: np.asarray(w[name], dtype=np.float64)
    return relu_squared(np.asarray(h, dtype=np.float64) @ f64("up").T + f64("up.b")) @ f64("down").T + f64("down.b")


def route(h, w_router, top):
    """(chosen experts [T, top], their weights [T, top]): scores are sigmoids of the router's products, the `top`
    largest are chosen (the lower index on a tie) and keep their scores as they are."""
    z = np.asarray(h, dtype=np.float64) @ np.asarray(w_router, dtype=np.float64).T
    s = 1.0 / (1.0 + np.exp(-z))
    order = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return order, np.take_along_axis(s, order, axis=-1)


def routed_feed_forward(h, w, experts, top):
    """Sum over a token's chosen experts of W_down,e relu(W_up,e (s_e h))^2: the score scales what goes in."""
    h = np.asarray(h, dtype=np.float64)
    ids, wts = route(h, w["router"], top)
    out = np.zeros((h.shape[0], np.asarray(w["e0.down"]).shape[0]))
    for t in range(h.shape[0]):
        for k in range(top):
            e = int(ids[t, k])
            up = np.asarray(w[f"e{e}.up"], dtype=np.float64)
            down = np.asarray(w[f"e{e}.down"], dtype=np.float64)
            out[t] += down @ relu_squared(up @ (wts[t, k] * h[t]))
    return out


def _sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence from position 0 (and, on request, the stream after every run of a layer)."""
    eps = config["norm"]["eps"]
    emb = np.asarray(tensors["embed"], dtype=np.float64)
    x = layer_norm(emb[np.asarray(tokens)], tensors["embed.norm"], eps)
    seen = []
    for i, layer in enumerate(config["layers"]):
        src = i
        while config["layers"][src].get("weights_of") is not None:       # a layer that borrows another layer's tensors
            src = config["layers"][src]["weights_of"]
        p = f"l{src}."
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        x = x + latent_attention(layer_norm(x, tensors[p + "norm1"], eps), _sub(tensors, p + "mix."), layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            hh = layer_norm(x, tensors[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                x = x + dense_feed_forward(hh, _sub(tensors, p + "mlp."))
            elif mlp["kind"] == "moe":
                x = x + routed_feed_forward(hh, _sub(tensors, p + "mlp."), mlp["router"]["experts"], mlp["router"]["top"])
            else:
                raise ValueError(mlp["kind"])
        seen.append(x.copy())
    logits = layer_norm(x, tensors["final.norm"], eps) @ emb.T
    return (logits, np.stack(seen)) if return_layers else logits


# ---- test models: random weights and a file of them -----------------------------------------------------------------
def _to_bf16_values(a):
    """Float32 values rounded to the nearest value that has 8 significant bits (ties to even), still as float32."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    bits = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return bits.astype(np.uint32).view(np.float32)


def random_weights(config, seed=0):
    """name -> float64 array for every tensor of `config`; all values fit bfloat16 exactly.  Layers that borrow another
    layer's tensors get none."""
    rng = np.random.default_rng(seed)
    d, out = int(config["width"]), {}

    def put(name, shape, std=None, mean=0.0):
        if std is None:
            std = 1.0 / math.sqrt(shape[-1]) if len(shape) > 1 else 0.5
        out[name] = _to_bf16_values(rng.standard_normal(shape) * std + mean).astype(np.float64).reshape(shape)

    put("embed", (int(config["vocab"]), d), 1.0)
    put("embed.norm", (d,), 0.1, 1.0)
    put("final.norm", (d,), 0.1, 1.0)
    for i, layer in enumerate(config["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", layer["mixer"]
        H, dn, dr, dv, r, rq = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
        put(p + "norm1", (d,), 0.1, 1.0)
        put(p + "mix.dq", (rq, d)); put(p + "mix.dq.norm", (rq,), 0.1, 1.0); put(p + "mix.uq", (H * (dn + dr), rq))
        put(p + "mix.dkv", (r + dr, d)); put(p + "mix.dkv.norm", (r,), 0.1, 1.0)
        put(p + "mix.uk", (H * dn, r)); put(p + "mix.uv", (H * dv, r)); put(p + "mix.o", (d, H * dv))
        mlp = layer.get("mlp")
        if not mlp:
            continue
        put(p + "norm2", (d,), 0.1, 1.0)
        if mlp["kind"] == "dense":
            f = int(mlp["ff"])
            put(p + "mlp.up", (f, d)); put(p + "mlp.up.b", (f,), 0.3); put(p + "mlp.down", (d, f)); put(p + "mlp.down.b", (d,), 0.3)
        else:
            f = int(mlp["expert"]["ff"])
            for e in range(int(mlp["router"]["experts"])):
                put(p + f"mlp.e{e}.up", (f, d)); put(p + f"mlp.e{e}.down", (d, f))
            put(p + "mlp.router", (int(mlp["router"]["experts"]), d), 4.0 / math.sqrt(d))
    return out


def write_bf16_file(path, tensors):
    """The tensors (bfloat16 values held in wider floats) as a safetensors file: 8 bytes of header length, the JSON header
    (name -> dtype, shape, data_offsets), then the data."""
    import json
    import struct
    header, chunks, at = {}, [], 0
    for name, a in tensors.items():
        raw = (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype("<u2").tobytes()
        header[name] = {"dtype": "BF16", "shape": list(np.shape(a)), "data_offsets": [at, at + len(raw)]}
        chunks.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + b"".join(chunks))
