"""Each kernel behind the hybrid decoder's parts alone, against the same operation written out in 64-bit torch, at sizes
that are not an engine's: attention with a cap, sinks, chunks or a window and values of their own width (the plain and
the tensor-core kernels, prompt rows after a cached prefix and one-token rows cut into slices, pages shuffled and unused
rows poisoned); the state-space layer's convolution, recurrence and gated norm across several steps; the router, the
sort by expert and the experts' products for few and for many rows; the gated epilogues with GELU."""
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from ghost_infer_b200.cache.sequence_cache import LayerMemory
from ghost_infer_b200.kernels import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def step_of(q_lens, pos0, slots):
    """What the kernels read of a step, on the device."""
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    positions = np.concatenate([np.arange(p, p + n) for p, n in zip(pos0, q_lens)]).astype(np.int32)
    token_slots = np.concatenate([np.full(n, s) for s, n in zip(slots, q_lens)]).astype(np.int32)
    t = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)
    return SimpleNamespace(n_seqs=len(q_lens), n_tokens=int(sum(q_lens)), max_q_len=int(max(q_lens)),
                           max_kv_len=int(max(p + n for p, n in zip(pos0, q_lens))), is_decode=max(q_lens) == 1,
                           cu_seqlens=t(cu), positions=t(positions), token_slots=t(token_slots), seq_slots=t(slots),
                           seq_pos0=t(pos0), seq_lens=t([p + n for p, n in zip(pos0, q_lens)]), sm_count=148)


def paged(k_dense, v_dense, lens, seed=0):
    """Dense [B, S, G, d] keys and values into shuffled pages; unused rows and pages hold NaN."""
    B, S, G, dk = k_dense.shape
    dv = v_dense.shape[3]
    per = (S + 63) // 64
    total = B * per + 4
    order = (torch.randperm(total - 1, generator=torch.Generator().manual_seed(seed)) + 1).tolist()
    kc = torch.full((total, G, 64, dk), float("nan"), dtype=k_dense.dtype, device=DEV)
    vc = torch.full((total, G, 64, dv), float("nan"), dtype=k_dense.dtype, device=DEV)
    kc[0], vc[0] = 0, 0
    bt = torch.zeros((B, per), dtype=torch.int32)
    it = iter(order)
    for b in range(B):
        for p in range((lens[b] + 63) // 64):
            page = next(it)
            bt[b, p] = page
            n = min(64, lens[b] - p * 64)
            kc[page, :, :n] = k_dense[b, p * 64:p * 64 + n].transpose(0, 1)
            vc[page, :, :n] = v_dense[b, p * 64:p * 64 + n].transpose(0, 1)
    return kc, vc, bt.to(DEV)


def attention_reference(q, k, v, pos0, q_lens, scale, cap, sinks, chunk, window):
    """q [T, H, dk] (flat over sequences), k, v [B, S, G, d] in 64-bit; returns [T, H * dv]."""
    H, G = q.shape[1], k.shape[2]
    out, at = [], 0
    for b, (p0, n) in enumerate(zip(pos0, q_lens)):
        for i in range(n):
            pos = p0 + i
            lo = 0
            if window:
                lo = max(lo, pos - window + 1)
            if chunk:
                lo = max(lo, pos // chunk * chunk)
            row = []
            for h in range(H):
                g = h // (H // G)
                s = (k[b, lo:pos + 1, g] @ q[at + i, h]) * scale
                if cap:
                    s = cap * torch.tanh(s / cap)
                top = s.max() if sinks is None else torch.maximum(s.max(), sinks[h])
                e = torch.exp(s - top)
                denom = e.sum() + (torch.exp(sinks[h] - top) if sinks is not None else 0.0)
                row.append((e / denom) @ v[b, lo:pos + 1, g])
            out.append(torch.cat(row))
        at += n
    return torch.stack(out)


CASES = [
    # H, G, dk, dv, cap, sinks, chunk, window
    (4, 2, 64, 56, 30.0, True, 100, None),
    (6, 2, 40, 72, None, True, None, 70),
    (3, 3, 128, 128, 5.0, False, 33, None),
    (8, 1, 24, 8, None, False, None, None),
    (4, 2, 64, 64, 12.0, True, 150, None),     # equal sizes of 64 or 128: the tcgen05 prompt kernel
    (2, 1, 128, 128, None, True, None, 90),
]


@pytest.mark.parametrize("dtype,tc", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
@pytest.mark.parametrize("case", CASES)
def test_attention_general_prompt_rows_and_one_token_rows(case, dtype, tc):
    H, G, dk, dv, cap, with_sinks, chunk, window = case
    g = torch.Generator().manual_seed(H * 100 + dk)
    q_lens, pos0 = [70, 1, 129], [60, 0, 131]          # after a cached prefix, a first token, across page borders
    lens = [p + n for p, n in zip(pos0, q_lens)]
    B, S = len(lens), max(lens)
    k = torch.randn(B, S, G, dk, generator=g).to(dtype)
    v = torch.randn(B, S, G, dv, generator=g).to(dtype)
    kc, vc, bt = paged(k.to(DEV), v.to(DEV), lens)
    sinks = torch.randn(H, generator=g) if with_sinks else None
    scale = 1.7 / math.sqrt(dk)
    mem = LayerMemory(kc, vc, bt, window, True, None, chunk)
    old = ops.TUNE["attn_general_tc"]
    ops.TUNE["attn_general_tc"] = tc
    try:
        for lens_q, p0s in ((q_lens, pos0), ([1, 1, 1], [n - 1 for n in lens])):
            T = sum(lens_q)
            q = torch.randn(T, H, dk, generator=g).to(dtype)
            qkv = torch.zeros(T, H * dk + G * dk + G * dv, dtype=dtype, device=DEV)
            qkv[:, :H * dk] = q.reshape(T, H * dk).to(DEV)
            step = step_of(lens_q, p0s, [0, 1, 2])
            out = torch.empty(T, H * dv, dtype=dtype, device=DEV)
            ops.attention_general(qkv, mem, step, H, G, dk, dv, scale, out, window=window, chunk=chunk, softcap=cap or 0.0,
                                  sinks=sinks.to(DEV) if sinks is not None else None)
            want = attention_reference(q.double(), k.double(), v.double(), p0s, lens_q, scale, cap,
                                       sinks.double() if sinks is not None else None, chunk, window)
            err = (out.double().cpu() - want).abs().max().item()
            assert np.isfinite(err) and err < (2e-5 if dtype == torch.float32 else 0.03), f"{case} {dtype} tc={tc}: {err}"
    finally:
        ops.TUNE["attn_general_tc"] = old


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_values_blended_and_stored(dtype):
    g = torch.Generator().manual_seed(1)
    H, G, dk, dv, T = 3, 2, 16, 24, 70
    qkv = torch.randn(T, H * dk + G * dk + G * dv, generator=g).to(dtype).to(DEV)
    first = torch.randn(T, G * dv, generator=g).to(dtype).to(DEV)
    lam = torch.tensor([0.3], device=DEV)
    kc = torch.zeros(4, G, 64, dk, dtype=dtype, device=DEV)
    vc = torch.zeros(4, G, 64, dv, dtype=dtype, device=DEV)
    bt = torch.tensor([[3, 1]], dtype=torch.int32, device=DEV)
    step = step_of([T], [20], [0])
    before = qkv.clone()
    copy = torch.empty(T, G * dv, dtype=dtype, device=DEV)
    ops.kv_store(qkv, step.positions, step.token_slots, LayerMemory(kc, vc, bt, None, True, None), H, G, dk, dv, first, lam, copy)
    v0 = before[:, (H + G) * dk:]
    assert torch.equal(copy, v0) and torch.equal(qkv[:, :(H + G) * dk], before[:, :(H + G) * dk])
    mixed = (0.7 * v0.double() + 0.3 * first.double())
    assert (qkv[:, (H + G) * dk:].double() - mixed).abs().max() < (1e-6 if dtype == torch.float32 else 0.02)
    for t in (0, 43, 44, T - 1):                   # position 20 + t: page 3 up to position 63, then page 1
        pos = 20 + t
        page, off = (3, pos) if pos < 64 else (1, pos - 64)
        assert torch.equal(kc[page, :, off].reshape(-1), before[t, H * dk:(H + G) * dk])
        assert torch.equal(vc[page, :, off].reshape(-1), qkv[t, (H + G) * dk:])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(3, 20, 24, 1, 3, 1), (4, 8, 128, 2, 4, 2), (2, 40, 70, 2, 2, 5), (1, 16, 300, 1, 1, 1)])
def test_state_space_steps_across_cuts_and_batches(sizes, dtype):
    heads, P, N, G, taps, parts = sizes
    g = torch.Generator().manual_seed(heads * 7 + N)
    inner, ch = heads * P, heads * P + 2 * G * N
    width = 2 * inner + 2 * G * N + heads
    lens = [37, 5]
    proj = [(torch.randn(n, width, generator=g) * 0.7).to(dtype) for n in lens]
    conv_w = (torch.randn(ch, taps, generator=g) * 0.5).to(dtype)
    conv_b = (torch.randn(ch, generator=g) * 0.2).to(dtype)
    dt_bias, a_log, d_skip = (torch.randn(heads, generator=g) * 0.5 for _ in range(3))
    norm_w = (1 + 0.1 * torch.randn(inner, generator=g)).to(dtype)
    s_floats = heads * N * P
    state = torch.zeros(4, s_floats + (taps - 1) * ch, device=DEV)

    def reference(pr):
        pr = pr.double()
        T = pr.shape[0]
        z, xbc, dt = pr[:, :inner], pr[:, inner:inner + ch], pr[:, inner + ch:]
        pad = torch.cat([torch.zeros(taps - 1, ch, dtype=torch.float64), xbc])
        conv = torch.stack([(pad[t:t + taps].T * conv_w.double()).sum(1) + conv_b.double() for t in range(T)])
        conv = torch.nn.functional.silu(conv).to(dtype).double()          # the kernel hands its result on in the rows' type
        x, Bm, Cm = conv[:, :inner].reshape(T, heads, P), conv[:, inner:inner + G * N].reshape(T, G, N), conv[:, inner + G * N:].reshape(T, G, N)
        dt = torch.nn.functional.softplus(dt + dt_bias.double())
        y = torch.zeros(T, heads, P, dtype=torch.float64)
        for h in range(heads):
            S = torch.zeros(N, P, dtype=torch.float64)
            for t in range(T):
                S = torch.exp(-torch.exp(a_log[h].double()) * dt[t, h]) * S + dt[t, h] * torch.outer(Bm[t, h // (heads // G)], x[t, h])
                y[t, h] = S.T @ Cm[t, h // (heads // G)] + d_skip[h].double() * x[t, h]
        y = y.reshape(T, inner) * torch.nn.functional.silu(z)
        y = y.reshape(T, parts, inner // parts)
        y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + 1e-5)
        return y.reshape(T, inner) * norm_w.double()

    want = [reference(p) for p in proj]
    # sequence 0 in slot 2 cut into 1 + 20 + 16 tokens, sequence 1 in slot 0 joining at the second step
    got = {0: [], 1: []}
    for entries in ([(0, 0, 1)], [(0, 1, 21), (1, 0, 5)], [(0, 21, 37)]):
        rows = torch.cat([proj[s][a:b] for s, a, b in entries]).to(DEV)
        step = step_of([b - a for _, a, b in entries], [a for _, a, _ in entries], [2 if s == 0 else 0 for s, _, _ in entries])
        xbc = ops.mamba2_conv(rows, conv_w.to(DEV), conv_b.to(DEV), state, step, inner, ch, taps, s_floats)
        y = ops.mamba2_scan(xbc, rows, dt_bias.to(DEV), a_log.to(DEV), d_skip.to(DEV), state, step, heads, P, N, G, taps)
        out = ops.mamba2_gate_norm(y, rows, norm_w.to(DEV), parts, 1e-5, dtype)
        at = 0
        for s, a, b in entries:
            got[s].append(out[at:at + b - a])
            at += b - a
    for s in (0, 1):
        err = (torch.cat(got[s]).double().cpu() - want[s]).abs().max().item()
        assert err < (2e-4 if dtype == torch.float32 else 0.06), f"{sizes} {dtype} sequence {s}: {err}"
    assert state[1].abs().max() == 0 and state[3].abs().max() == 0          # other slots' rows untouched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,top,d,f", [(5, 4, 4, 40, 24), (9, 37, 3, 64, 16), (700, 6, 2, 72, 40), (1200, 3, 1, 32, 8)])
def test_router_sort_and_expert_products(T, E, top, d, f, dtype):
    g = torch.Generator().manual_seed(T + E)
    h = torch.randn(T, d, generator=g).to(dtype)
    wr = (torch.randn(E, d, generator=g) * 0.4).to(dtype)
    wsg = (torch.randn(d, generator=g) * 0.3).to(dtype)
    gate, up = (torch.randn(E, f, d, generator=g) * 0.2).to(dtype), (torch.randn(E, f, d, generator=g) * 0.2).to(dtype)
    down = (torch.randn(E, d, f, generator=g) * 0.2).to(dtype)
    ids, wts, sg = ops.moe_route(h.to(DEV), wr.to(DEV), top, wsg.to(DEV))
    logits = h.double() @ wr.double().T
    order = torch.argsort(-logits, dim=1, stable=True)[:, :top]
    gaps = torch.sort(logits, dim=1, descending=True).values
    sure = (gaps[:, :top] - gaps[:, 1:top + 1]).min(dim=1).values > 1e-3 if top < E else torch.ones(T, dtype=torch.bool)
    assert torch.equal(ids.cpu().long()[sure], order[sure])
    chosen = torch.gather(logits, 1, ids.cpu().long())
    assert (wts.cpu().double() - torch.softmax(chosen, 1)).abs().max() < 1e-5
    assert (sg.cpu().double() - torch.sigmoid(h.double() @ wsg.double())).abs().max() < 1e-5
    offsets, perm, inv = ops.moe_plan(ids, E)
    flat = ids.cpu().reshape(-1)
    want_perm = torch.argsort(flat, stable=True)
    assert torch.equal(perm.cpu().long(), want_perm) and torch.equal(perm[inv.long()].cpu(), torch.arange(T * top, dtype=torch.int32))
    assert offsets.cpu().tolist() == np.concatenate([[0], np.cumsum(np.bincount(flat.numpy(), minlength=E))]).tolist()
    assert torch.equal(ops.moe_gather_rows(h.to(DEV), perm, top).cpu(), h[(want_perm // top)])
    for interleaved in ((False, True) if f % 8 == 0 else (False,)):
        if interleaved:
            gu = torch.stack([gate.reshape(E, f // 8, 8, d), up.reshape(E, f // 8, 8, d)], dim=2).reshape(E, 2 * f, d)
        else:
            gu = torch.cat([gate, up], dim=1)
        out = ops.moe_experts(h.to(DEV), gu.contiguous().to(DEV), down.to(DEV), offsets, perm, top, interleaved)
        x = torch.zeros(T, d, device=DEV)
        shared = torch.randn(T, d, generator=g).to(DEV)
        ops.moe_combine(x, out, inv, wts, shared, sg)
        want = torch.zeros(T, d, dtype=torch.float64)
        for t in range(T):
            for k in range(top):
                e = int(ids[t, k])
                a = (torch.nn.functional.silu(gate[e].double() @ h[t].double()) * (up[e].double() @ h[t].double())).to(dtype).double()
                want[t] += wts[t, k].double().cpu() * (down[e].double() @ a)
        want += sg.cpu().double()[:, None] * shared.cpu().double()
        err = (x.cpu().double() - want).abs().max().item()
        assert err < (2e-5 if dtype == torch.float32 else 0.02), f"interleaved={interleaved}: {err}"


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


@pytest.mark.parametrize("rows", [3, 40, 200])
def test_gelu_in_the_gated_epilogues(rows):
    g = torch.Generator().manual_seed(rows)
    d, f = 96, 80
    h = torch.randn(rows, d, generator=g).to(torch.bfloat16)
    gate, up = (torch.randn(f, d, generator=g) * 0.3).to(torch.bfloat16), (torch.randn(f, d, generator=g) * 0.3).to(torch.bfloat16)
    w = torch.stack([gate.reshape(f // 8, 8, d), up.reshape(f // 8, 8, d)], dim=1).reshape(2 * f, d).contiguous()
    want = gelu_tanh(h.double() @ gate.double().T) * (h.double() @ up.double().T)
    got = ops.swiglu_interleaved(h.to(DEV), w.to(DEV), "gelu_tanh")
    assert (got.double().cpu() - want).abs().max() < 0.03 * float(want.abs().max())
    silu = torch.nn.functional.silu(h.double() @ gate.double().T) * (h.double() @ up.double().T)
    assert (ops.swiglu_interleaved(h.to(DEV), w.to(DEV)).double().cpu() - silu).abs().max() < 0.03 * float(silu.abs().max())
    for dt in (torch.float32, torch.bfloat16):
        gu = torch.cat([h.double() @ gate.double().T, h.double() @ up.double().T], dim=1).to(dt)
        ref = gelu_tanh(gu[:, :f].double()) * gu[:, f:].double()
        out = ops.act_mul(gu.to(DEV), "gelu_tanh")
        assert (out.double().cpu() - ref).abs().max() < (1e-5 if dt == torch.float32 else 0.02) * max(1.0, float(ref.abs().max()))
    ops.check_status()


def test_embedding_times_a_constant():
    table = torch.randn(50, 24).to(torch.bfloat16).to(DEV)
    tokens = torch.tensor([3, 49, 0, 3], dtype=torch.int32, device=DEV)
    assert torch.equal(ops.embed(table, tokens, scale=0.5), table[tokens.long()].float() * 0.5)
    assert torch.equal(ops.embed(table, tokens), table[tokens.long()].float())


def test_experts_expert_by_expert_on_tensor_cores():
    """A prompt step's way through the experts (rows gathered in sorted order, then each expert's stretch through the
    tensor-core products) against the grouped kernel on the same rows; stretches of fewer and of more than 64 rows."""
    g = torch.Generator().manual_seed(9)
    T, E, top, d, f = 900, 7, 1, 72, 40
    h = torch.randn(T, d, generator=g).to(torch.bfloat16).to(DEV)
    wr = torch.randn(E, d, generator=g) * 0.4
    wr[5] *= 0.05                                      # an expert that few tokens choose: a short stretch
    gate, up = (torch.randn(E, f, d, generator=g) * 0.2).to(torch.bfloat16), (torch.randn(E, f, d, generator=g) * 0.2).to(torch.bfloat16)
    gu = torch.stack([gate.reshape(E, f // 8, 8, d), up.reshape(E, f // 8, 8, d)], dim=2).reshape(E, 2 * f, d).contiguous().to(DEV)
    down = (torch.randn(E, d, f, generator=g) * 0.2).to(torch.bfloat16).to(DEV)
    ids, wts, _ = ops.moe_route(h, wr.to(torch.bfloat16).to(DEV), top)
    offsets, perm, inv = ops.moe_plan(ids, E)
    counts = np.diff(offsets.cpu().numpy())
    assert counts.min() <= 64 < counts.max()
    want = ops.moe_experts(h, gu, down, offsets, perm, top, True)
    got = ops.moe_experts_by_expert(ops.moe_gather_rows(h, perm, top), gu, down, offsets.cpu().tolist())
    ops.check_status()
    assert (got - want).abs().max().item() < 0.02 * want.abs().max().item()
