"""The kernels of the Rirulix design's mechanisms, each alone against plain PyTorch in float64 with
inputs made so that a fault shows: a far key that carries the whole weight among hundreds, keys just
inside and just outside a window and the kept first tokens, at page borders, in runs and for single
tokens; a recurrent state carried over portions; experts chosen two at a time."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

from qwen25vl_lite.engine.runner import HostStep, KVStep
from qwen25vl_lite.ops import attention as attention_ops
from qwen25vl_lite.ops import kernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def group_norm(v, w, groups, eps):
    n, d = v.shape
    x = v.double().reshape(n, groups, d // groups)
    return (x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)).reshape(n, d) * w.double()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,groups,dgroups", [(96, 3, 3), (384, 1, 4), (1024, 8, 2)])
def test_add_norm_groups(dtype, hidden, groups, dgroups):
    g = torch.Generator(device=DEV).manual_seed(1)
    n = 9
    x = torch.randn(n, hidden, generator=g, device=DEV)
    delta = (torch.randn(n, hidden, generator=g, device=DEV) * 3).to(dtype)
    dw, w = torch.rand(hidden, generator=g, device=DEV) + 0.5, torch.rand(hidden, generator=g, device=DEV) + 0.5
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    # the update normalised on its way in, then the stream normalised for the next sublayer
    x1, out = x.clone(), torch.empty(n, hidden, dtype=dtype, device=DEV)
    kernels.add_norm_groups(x1, delta, dw, 1e-5, dgroups, w, 1e-6, groups, out)
    want_x = x.double() + group_norm(delta, dw, dgroups, 1e-5)
    assert (x1.double() - want_x).abs().max() < 1e-5
    assert (out.double() - group_norm(want_x, w, groups, 1e-6)).abs().max() < tol
    # chosen rows only: the stream stays as it is
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV)
    x2, out2 = x.clone(), torch.empty(3, hidden, dtype=dtype, device=DEV)
    kernels.add_norm_groups(x2, delta, dw, 1e-5, dgroups, w, 1e-6, groups, out2, rows)
    assert torch.equal(x2, x)
    assert (out2.double() - group_norm(want_x, w, groups, 1e-6)[rows.long()]).abs().max() < tol
    # an update that is added as it is, and none at all
    x3, out3 = x.clone(), torch.empty(n, hidden, dtype=dtype, device=DEV)
    kernels.add_norm_groups(x3, delta, None, 0.0, 1, w, 1e-6, groups, out3)
    assert (x3.double() - (x.double() + delta.double())).abs().max() < 1e-5
    x4 = x.clone()
    kernels.add_norm_groups(x4, None, None, 0.0, 1, w, 1e-6, groups, out3)
    assert torch.equal(x4, x) and (out3.double() - group_norm(x, w, groups, 1e-6)).abs().max() < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_position_norm(dtype):
    g = torch.Generator(device=DEV).manual_seed(2)
    vocab, places, hidden, groups = 50, 40, 192, 4
    table = torch.randn(vocab, hidden, generator=g, device=DEV).to(dtype)
    pos = torch.randn(places, hidden, generator=g, device=DEV).to(dtype)
    w = torch.rand(hidden, generator=g, device=DEV) + 0.5
    ids = torch.tensor([3, 49, 0, 3, 17], dtype=torch.int32, device=DEV)
    at = torch.tensor([0, 39, 5, 6, 7], dtype=torch.int32, device=DEV)
    x = torch.empty(5, hidden, device=DEV)
    kernels.embed_position_norm(table, pos, ids, at, w, 1e-6, groups, x)
    want = group_norm(table[ids.long()].double() + pos[at.long()].double(), w, groups, 1e-6)
    assert (x.double() - want).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_glu_clamped(dtype):
    g = torch.Generator(device=DEV).manual_seed(3)
    gu = (torch.randn(11, 2 * 40, generator=g, device=DEV) * 3).to(dtype)
    out = torch.empty(11, 40, dtype=dtype, device=DEV)
    kernels.glu_clamped(gu, out, 1.25, 1.702)
    a, b = gu[:, :40].double().clamp(max=1.25), gu[:, 40:].double().clamp(-1.25, 1.25)
    want = a * torch.sigmoid(1.702 * a) * (b + 1)
    assert (out.double() - want).abs().max() < (1e-6 if dtype == torch.float32 else 2e-2)
    assert (a == 1.25).any() and (b == -1.25).any()                  # the clamps were reached


# ---- the gated linear recurrence ----------------------------------------------------------------------


def recurrence_reference(yx, width, conv_w, conv_b, ra, ra_b, ri, ri_b, lam, gain):
    """One request's whole sequence in float64."""
    y, xin = yx[:, :width].double(), yx[:, width:].double()
    n, taps = xin.shape[0], conv_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, width, dtype=torch.float64, device=yx.device), xin])
    u = sum(padded[j:j + n] * conv_w[:, j].double() for j in range(taps)) + conv_b.double()
    blocks = ra.shape[0]
    ub = u.reshape(n, blocks, -1)
    gate = lambda m, b: torch.sigmoid(torch.einsum("boi,nbi->nbo", m.double(), ub) + b.double()).reshape(n, width)
    a = torch.exp(-gain * gate(ra, ra_b) * torch.nn.functional.softplus(lam.double()))
    s, out = torch.zeros(width, dtype=torch.float64, device=yx.device), []
    for t in range(n):
        s = a[t] * s + torch.sqrt(1 - a[t] ** 2) * gate(ri, ri_b)[t] * u[t]
        out.append(s * torch.nn.functional.gelu(y[t], approximate="tanh"))
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,blocks,taps", [(64, 4, 3), (176, 1, 2), (96, 3, 1), (256, 2, 4), (66, 3, 2)])
def test_recurrence_in_portions_with_state(dtype, width, blocks, taps):
    """Two requests of unequal length in three steps (portions of 1, 2 and many tokens, the second
    request absent from the middle step), in slots 2 and 0 of three: the state carries S and the
    convolution's last inputs, and the result is the whole sequence's.  The last step's 260 tokens
    are scanned in nine chunks beside an entry of one chunk, and its gates come from the tiled
    product where the small steps' come from the one that holds the whole depth at once."""
    g = torch.Generator(device=DEV).manual_seed(4)
    rnd = lambda *shape, scale=1.0: torch.randn(*shape, generator=g, device=DEV) * scale
    bw = width // blocks
    conv_w, conv_b = rnd(width, taps, scale=0.5), rnd(width, scale=0.1)
    ra, ra_b, ri, ri_b, lam = rnd(blocks, bw, bw, scale=0.3), rnd(blocks, bw), rnd(blocks, bw, bw, scale=0.3), rnd(blocks, bw), rnd(width)
    lens = {"a": 263, "b": 9}
    yx = {k: rnd(n, 2 * width).to(dtype) for k, n in lens.items()}
    want = {k: recurrence_reference(yx[k], width, conv_w, conv_b, ra, ra_b, ri, ri_b, lam, 8.0) for k in lens}
    state = torch.zeros(3, taps, width, device=DEV)
    slot = {"a": 2, "b": 0}
    done = {"a": 0, "b": 0}
    got = {"a": [], "b": []}
    for step in ({"a": 1, "b": 2}, {"a": 2}, {"a": 260, "b": 7}):
        names = list(step)
        rows = torch.cat([yx[k][done[k]:done[k] + step[k]] for k in names])
        n = rows.shape[0]
        cu = torch.tensor(np.concatenate([[0], np.cumsum([step[k] for k in names])]), dtype=torch.int32, device=DEV)
        token_seq = torch.tensor(np.repeat(np.arange(len(names)), [step[k] for k in names]), dtype=torch.int32, device=DEV)
        slots = torch.tensor([slot[k] for k in names], dtype=torch.int32, device=DEV)
        u, a, bx = (torch.empty(n, width, device=DEV) for _ in range(3))
        out = torch.empty(n, width, dtype=dtype, device=DEV)
        kernels.rglru_conv(rows, width, conv_w, conv_b, state, token_seq, cu, slots, u)
        kernels.rglru_gates(u, ra, ra_b, ri, ri_b, lam, 8.0, a, bx)
        kernels.rglru_scan(a, bx, rows, 0, width, state, cu, slots, out, len(names), max(step.values()))
        at = 0
        for k in names:
            got[k].append(out[at:at + step[k]])
            at += step[k]
            done[k] += step[k]
    assert state[1].abs().max() == 0                                   # nobody's slot stays untouched
    for k in lens:
        err = (torch.cat(got[k]).double() - want[k]).abs().max()
        assert err < (2e-5 if dtype == torch.float32 else 3e-2), (k, float(err))


# ---- the routed feed-forward ------------------------------------------------------------------------------


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,experts,top,hidden,ff", [(1, 4, 1, 64, 24), (7, 6, 2, 96, 40), (150, 5, 3, 128, 48), (300, 8, 1, 352, 72),
                                                     (700, 4, 1, 72, 40), (33, 3, 2, 100, 30), (600, 2, 1, 44, 20),
                                                     (1300, 4, 1, 72, 40), (1100, 16, 2, 64, 24)])
def test_routed_experts(dtype, n, experts, top, hidden, ff, monkeypatch):
    """From one token to hundreds per expert (row tiles of 16, 64 and 128), one to three choices, sizes
    that the tensor-core product does not take (a width that is no multiple of 8), and steps of more
    than a thousand pairs.  Long bfloat16 steps whose sizes allow it take the grouped tcgen05 product."""
    from qwen25vl_lite.parts import feed_forward
    from qwen25vl_lite.parts.feed_forward import RoutedGLU

    monkeypatch.setattr(feed_forward, "TCGEN05_MIN_WIDTH", 64)          # the tcgen05 grouped product at these small widths too
    g = torch.Generator(device=DEV).manual_seed(5)
    rnd = lambda *shape, scale=1.0: torch.randn(*shape, generator=g, device=DEV) * scale
    part = RoutedGLU(hidden, experts, top, ff, limit=1.5, shared_size=32, shared_limit=0.75)
    tensors = {"router": rnd(experts, hidden, scale=0.2)}
    for e in range(experts):
        tensors.update({f"e{e}.gate": rnd(ff, hidden, scale=0.2), f"e{e}.up": rnd(ff, hidden, scale=0.2), f"e{e}.down": rnd(hidden, ff, scale=0.2)})
    tensors.update({"shared.gate": rnd(32, hidden, scale=0.2), "shared.up": rnd(32, hidden, scale=0.2), "shared.down": rnd(hidden, 32, scale=0.2),
                    "shared.sg": rnd(1, hidden, scale=0.2)})
    tensors = {k: v.to(dtype).float() for k, v in tensors.items()}      # what bfloat16 can hold, in both runs
    part.load(tensors, DEV, dtype)
    h = rnd(n, hidden).to(dtype)
    out = part.forward(SimpleNamespace(dtype=dtype), h)
    x, w = h.double(), {k: v.double() for k, v in tensors.items()}

    def expert(a, p, limit):
        gate = (a @ w[p + "gate"].T).clamp(max=limit)
        up = (a @ w[p + "up"].T).clamp(-limit, limit)
        return (gate * torch.sigmoid(1.702 * gate) * (up + 1)) @ w[p + "down"].T

    scores = torch.sigmoid(x @ w["router"].T)
    want = torch.sigmoid(x @ w["shared.sg"].T) * expert(x, "shared.", 0.75)
    for t in range(n):
        for e in torch.topk(scores[t], top).indices.tolist():
            want[t] += expert(scores[t, e] * x[t:t + 1], f"e{e}.", 1.5)[0]
    err = (out.double() - want).abs().max()
    assert err < (2e-5 if dtype == torch.float32 else 0.05 * float(want.abs().max())), float(err)


# ---- attention ---------------------------------------------------------------------------------------------


def attention_case(dtype, nq, nkv, dk, dv, page_size, window, keep, entries, seed, peaks):
    """``entries``: (tokens already in the cache, tokens of this step) per request.  ``peaks``: for
    entry e, query token t (index in the step) and head h, the key j whose score is made to stand out
    by s: q = s * unit, k_j = unit.  Builds pages in a shuffled order and returns the kernel's
    output beside the float64 reference."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    rnd = lambda *shape, scale=1.0: torch.randn(*shape, generator=g, device=DEV) * scale
    group = nq // nkv
    total = [s + n for s, n in entries]
    ks = [rnd(t, nkv, dk, scale=0.3) for t in total]
    vs = [rnd(t, nkv, dv) for t in total]
    qs = [rnd(n, nq, dk, scale=0.3) for _, n in entries]
    for e, t, h, j, strength in peaks:
        unit = torch.zeros(dk, device=DEV)
        unit[(7 * j + h) % dk] = 1.0
        ks[e][j, h // group] = unit * 4.0
        qs[e][t, h] = unit * strength
    to = lambda x: x.to(dtype)
    ks, vs, qs = [to(k) for k in ks], [to(v) for v in vs], [to(q) for q in qs]
    pages_needed = [-(-t // page_size) for t in total]
    n_pages = sum(pages_needed) + 3
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    k_pages = torch.zeros(n_pages, nkv, page_size, dk, dtype=dtype, device=DEV)
    v_pages = torch.zeros(n_pages, nkv, page_size, dv, dtype=dtype, device=DEV)
    width = max(pages_needed)
    table = torch.zeros(len(entries), width, dtype=torch.int32)
    for e, t in enumerate(total):
        for p in range(pages_needed[e]):
            page = order.pop()
            table[e, p] = page
            lo, hi = p * page_size, min((p + 1) * page_size, t)
            k_pages[page, :, :hi - lo] = ks[e][lo:hi].transpose(0, 1)
            v_pages[page, :, :hi - lo] = vs[e][lo:hi].transpose(0, 1)
    q_lens, starts = [n for _, n in entries], [s for s, _ in entries]
    n_tokens = sum(q_lens)
    qkv = torch.zeros(n_tokens, nq * dk + nkv * dk + nkv * dv, dtype=dtype, device=DEV)
    qkv[:, :nq * dk] = torch.cat(qs).reshape(n_tokens, nq * dk)
    r1 = torch.rand(nq, generator=g, device=DEV) * 0.5
    r2 = torch.rand(nq, generator=g, device=DEV) * 2.0
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    ctx = SimpleNamespace(dtype=dtype, token_seq=i32(np.repeat(np.arange(len(entries)), q_lens)), cu_q=i32(np.concatenate([[0], np.cumsum(q_lens)])),
                          q_start_pos=i32(starts), n_seqs=len(entries), n_tokens=n_tokens, max_kv_len=max(total), max_q_len=max(q_lens))
    plan = {k: (i32(v) if len(v) else None) for k, v in attention_ops.plan_biased(HostStep(q_lens, starts, n_tokens, len(entries)), group, window or 0, keep).items()}
    kv = KVStep(k_pages, v_pages, None, table.to(DEV), page_size)
    out = attention_ops.attend_biased(ctx, plan, qkv, kv, nq, nkv, dk, dv, window, keep, 0.25, r1, r2)
    want = []
    for e, (s, n) in enumerate(entries):
        i = torch.arange(s, s + n, device=DEV)[:, None]
        j = torch.arange(s + n, device=DEV)[None, :]
        see = (j <= i) & (((i - j) < window) | (j < keep) if window else torch.ones_like(j <= i))
        for h in range(nq):
            sc = (qs[e][:, h].double() @ ks[e][:, h // group].double().T) * 0.25 - r1[h].double() * torch.log1p(r2[h].double() * (i - j).clamp(min=0))
            sc = torch.where(see, sc, torch.tensor(-float("inf"), dtype=torch.float64, device=DEV))
            want.append((e, h, torch.softmax(sc, dim=1) @ vs[e][:, h // group].double()))
    ref = torch.zeros(n_tokens, nq, dv, dtype=torch.float64, device=DEV)
    first = np.concatenate([[0], np.cumsum(q_lens)])
    for e, h, o in want:
        ref[first[e]:first[e + 1], h] = o
    return out.double().reshape(n_tokens, nq, dv), ref


SHAPES = [(6, 2, 64, 64), (4, 4, 32, 64), (6, 1, 128, 64), (3, 3, 48, 80), (8, 2, 64, 128)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,dk,dv", SHAPES)
def test_attention_edges_of_window_and_kept_tokens(dtype, nq, nkv, dk, dv):
    """Window 40, 3 kept tokens, pages of 16.  Peaked scores on the keys just inside the window
    (i - 39), just outside (i - 40: must not count), the last kept token (2) and the first not kept
    (3: hidden once the window has passed it), for tokens in a run and for single tokens, and on the
    query's own key."""
    window, keep = 40, 3
    entries = [(0, 100), (77, 1), (60, 31), (2, 1), (45, 1)]
    peaks = []
    for e, (s, n) in enumerate(entries):
        t = n - 1
        i = s + t
        for h, j in enumerate([i - 39, i - 40, 2, 3, i, i - 16]):
            if 0 <= j <= i and h < nq:
                peaks.append((e, t, h, j, 20.0))
    peaks += [(0, 50, 0, 11, 20.0), (0, 50, 1, 10, 20.0), (0, 42, 0, 3, 20.0), (0, 43, 1, 3, 20.0), (2, 3, 2, 32, 20.0), (2, 4, 2, 24, 20.0)]
    out, ref = attention_case(dtype, nq, nkv, dk, dv, 16, window, keep, entries, 6, peaks)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert (out - ref).abs().max() < tol, float((out - ref).abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,dk,dv", SHAPES[:3])
@pytest.mark.parametrize("page_size", [8, 16, 32])
def test_attention_far_key_among_hundreds(dtype, nq, nkv, dk, dv, page_size):
    """No window: 700 keys, and the whole weight of some queries on one key hundreds of tokens back
    (keys 0, 1, the last of a page, the first of the next), against the distance bias that grows
    with every token between them; a single token after 650 and a run after 300."""
    entries = [(650, 1), (300, 200), (0, 130)]
    peaks = [(0, 0, 0, 0, 40.0), (0, 0, 1, 1, 40.0), (0, 0, 2, page_size - 1, 40.0), (0, 0, 3, page_size, 40.0),
             (1, 199, 0, 5, 40.0), (1, 199, 1, 255, 40.0), (1, 0, 2, 17, 40.0), (1, 100, 3, 399, 40.0), (2, 129, 0, 0, 40.0), (2, 64, 1, 63, 40.0)]
    peaks = [p for p in peaks if p[2] < nq]
    out, ref = attention_case(dtype, nq, nkv, dk, dv, page_size, None, 0, entries, 7, peaks)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert (out - ref).abs().max() < tol, float((out - ref).abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_window_shorter_than_a_page_and_no_kept_tokens(dtype):
    entries = [(0, 70), (33, 1), (15, 2), (16, 1)]
    peaks = [(0, 69, 0, 65, 20.0), (0, 69, 1, 64, 20.0), (1, 0, 0, 29, 20.0), (1, 0, 1, 28, 20.0), (2, 1, 0, 12, 20.0), (2, 1, 1, 11, 20.0),
             (3, 0, 0, 12, 20.0), (3, 0, 1, 11, 20.0)]
    out, ref = attention_case(dtype, 4, 2, 64, 64, 16, 5, 0, entries, 8, peaks)
    assert (out - ref).abs().max() < (2e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_values_are_mixed_before_they_are_cached(dtype):
    g = torch.Generator(device=DEV).manual_seed(9)
    nq, nkv, dk, dv, ps, n = 4, 2, 32, 16, 8, 5
    qkv = torch.randn(n, nq * dk + nkv * dk + nkv * dv, generator=g, device=DEV).to(dtype)
    other = torch.randn(n, 100, generator=g, device=DEV).to(dtype)[:, 10:10 + nkv * dv]          # rows with a stride of their own
    k_pages = torch.zeros(6, nkv, ps, dk, dtype=dtype, device=DEV)
    v_pages = torch.zeros(6, nkv, ps, dv, dtype=dtype, device=DEV)
    slots = torch.tensor([5 * ps + 7, 2 * ps, 2 * ps + 1, 0, 3 * ps + 3], dtype=torch.int32, device=DEV)
    before = qkv.clone()
    kernels.kv_store_mix(qkv, other, 0.3, k_pages, v_pages, slots, nq, nkv, dk, dv, ps)
    mixed = 0.7 * before[:, (nq + nkv) * dk:].double() + 0.3 * other.double()
    for t, s in enumerate(slots.tolist()):
        assert torch.equal(k_pages[s // ps, :, s % ps].reshape(-1), before[t, nq * dk:(nq + nkv) * dk])
        assert (v_pages[s // ps, :, s % ps].reshape(-1).double() - mixed[t]).abs().max() < (1e-6 if dtype == torch.float32 else 2e-2)
    assert int((k_pages != 0).any(dim=-1).sum()) == n * nkv                          # nothing else was written
