"""The kernels of the Labolix design's mechanisms, each alone against plain float64 arithmetic, with
inputs made so that a fault shows: a far key that carries the whole weight among hundreds, keys just
inside and just outside a window, at page borders, in runs and for single tokens; a sink that takes
most of the weight; a retention state carried over portions and through slots that are used again."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

from plain import labolix as plain
from qwen25vl_lite.engine.runner import HostStep, KVStep
from qwen25vl_lite.ops import attention as attention_ops
from qwen25vl_lite.ops import kernels
from qwen25vl_lite.parts.position import rotary_frequencies

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [96, 130, 2048])
def test_dynamic_tanh_with_the_residual_update(dtype, hidden):
    g = torch.Generator(device=DEV).manual_seed(1)
    n = 7
    x = torch.randn(n, hidden, generator=g, device=DEV) * 2
    delta = torch.randn(n, hidden, generator=g, device=DEV).to(dtype)
    w, b = torch.rand(hidden, generator=g, device=DEV) + 0.5, torch.randn(hidden, generator=g, device=DEV)
    tol = 2e-6 if dtype == torch.float32 else 2e-2
    want_x = x.double() + delta.double()
    norm = lambda v: torch.tanh(0.37 * v) * w.double() + b.double()
    x1, out = x.clone(), torch.empty(n, hidden, dtype=dtype, device=DEV)
    kernels.add_dyt(x1, delta, w, b, 0.37, out)
    assert (x1.double() - want_x).abs().max() < 1e-6 and (out.double() - norm(want_x)).abs().max() < tol
    rows = i32([5, 0, 3])                       # chosen rows only: the stream stays as it is
    x2, out2 = x.clone(), torch.empty(3, hidden, dtype=dtype, device=DEV)
    kernels.add_dyt(x2, delta, w, b, 0.37, out2, rows)
    assert torch.equal(x2, x) and (out2.double() - norm(want_x)[rows.long()]).abs().max() < tol
    x3 = x.clone()                              # nothing to add
    kernels.add_dyt(x3, None, w, b, 0.37, out)
    assert torch.equal(x3, x) and (out.double() - norm(x.double())).abs().max() < tol


def test_softcap():
    logits = torch.linspace(-80, 80, 1001, device=DEV).reshape(7, 143).contiguous()
    want = 15.0 * torch.tanh(logits.double() / 15.0)
    kernels.softcap(logits, 15.0)
    assert (logits.double() - want).abs().max() < 2e-6 and logits.abs().max() < 15.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout,dims,width,scaling", [
    ("interleaved", 16, 32, {"kind": "wavelength", "factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}),
    ("halves", 24, 24, None), ("interleaved", 8, 8, {"kind": "ramp", "factor": 4.0, "original": 48, "fast": 8.0, "slow": 1.0}),
    ("halves", 6, 20, None)])
def test_rotation_of_part_of_a_head(dtype, layout, dims, width, scaling):
    """In place on the heads of a wider row, and from one strided buffer into another; positions up to thousands."""
    g = torch.Generator(device=DEV).manual_seed(2)
    freqs, magnitude = rotary_frequencies(dims, 1000.0, scaling)
    positions = i32([0, 1, 2, 47, 48, 49, 1000, 4095])
    n, heads, lead = positions.shape[0], 3, 5
    angles = kernels.rotary_angles(positions, torch.tensor(freqs, dtype=torch.float32, device=DEV), magnitude)
    rows = torch.randn(n, lead + heads * width + 7, generator=g, device=DEV).to(dtype)
    view = rows[:, lead:lead + heads * width].unflatten(1, (heads, width))
    want = plain.rotate(view.double().cpu().numpy(), positions.cpu().numpy(), freqs, magnitude, "interleaved" if layout == "interleaved" else "half")
    tol = 3e-4 if dtype == torch.float32 else 3e-2           # float32 angles at position 4095 carry 2e-4 of rounding
    other = torch.zeros(n, heads, width + 3, dtype=dtype, device=DEV)
    kernels.rotary_apply(view, other[:, :, 3:], heads, width, angles, layout)
    assert np.abs(other[:, :, 3:].double().cpu().numpy() - want).max() < tol and other[:, :, :3].abs().max() == 0
    before = rows.clone()
    kernels.rotary_apply(view, view, heads, width, angles, layout)
    assert np.abs(view.double().cpu().numpy() - want).max() < tol
    assert torch.equal(rows[:, :lead], before[:, :lead]) and torch.equal(rows[:, lead + heads * width:], before[:, lead + heads * width:])
    if width > dims:
        assert torch.equal(view[:, :, dims:], before[:, lead:lead + heads * width].unflatten(1, (heads, width))[:, :, dims:])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank,rot", [(40, 8), (64, 16), (200, 32), (24, 0)])
def test_latent_cache_row(dtype, rank, rot):
    g = torch.Generator(device=DEV).manual_seed(3)
    n, page_size, pages = 6, 4, 5
    freqs, magnitude = rotary_frequencies(rot, 500.0, None)
    positions = i32([3, 4, 5, 100, 0, 77])
    angles = kernels.rotary_angles(positions, torch.tensor(freqs, dtype=torch.float32, device=DEV), magnitude) if rot else None
    rows = torch.randn(n, 11 + rank + rot, generator=g, device=DEV).to(dtype) * 3
    x = rows[:, 11:]
    w = torch.rand(rank, generator=g, device=DEV) + 0.5
    cache = torch.zeros(pages, 1, page_size, rank + rot, dtype=dtype, device=DEV)
    slots = i32([17, 2, 3, 8, 0, 19])
    kernels.latent_store(x, rank, rot, w, 1e-5, angles, "interleaved", cache, slots)
    xd = x.double().cpu().numpy()
    want = np.concatenate([plain.rms_unit(xd[:, :rank], 1e-5) * w.double().cpu().numpy(),
                           plain.rotate(xd[:, None, rank:], positions.cpu().numpy(), freqs, magnitude, "interleaved")[:, 0]], axis=1)
    got = cache.reshape(pages * page_size, rank + rot).double().cpu().numpy()
    assert np.abs(got[slots.cpu().numpy()] - want).max() < (1e-4 if dtype == torch.float32 else 4e-2)
    untouched = np.setdiff1d(np.arange(pages * page_size), slots.cpu().numpy())
    assert np.abs(got[untouched]).max() == 0


# ---- attention with a sink; values inside the key rows -------------------------------------------------------


def sink_attention_case(dtype, nq, nkv, dk, dv, page_size, window, sink, latent, entries, seed, peaks, scale=0.25):
    """``entries``: (tokens already in the cache, tokens of this step) per request.  ``peaks``: (entry,
    query token of the step, head, key j, strength): that query's score on key j is made to stand out.
    ``latent``: one kv head whose value is the first dv channels of its key row.  Pages are handed out in
    a shuffled order.  Returns the kernels' output beside the float64 reference."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    rnd = lambda *shape, scale=1.0: torch.randn(*shape, generator=g, device=DEV) * scale
    group = nq // nkv
    total = [s + n for s, n in entries]
    ks = [rnd(t, nkv, dk, scale=0.3) for t in total]
    qs = [rnd(n, nq, dk, scale=0.3) for _, n in entries]
    for e, t, h, j, strength in peaks:
        unit = torch.zeros(dk, device=DEV)
        unit[dk - 1 - (7 * j + h) % (dk // 2)] = 1.0          # in the channels that are no value of a latent row
        ks[e][j, h // group, dk // 2:] = 0
        ks[e][j, h // group] += unit * 4.0
        qs[e][t, h] = unit * strength
    ks, qs = [k.to(dtype) for k in ks], [q.to(dtype) for q in qs]
    vs = [k[:, :, :dv] for k in ks] if latent else [rnd(t, nkv, dv).to(dtype) for t in total]
    pages_needed = [-(-t // page_size) for t in total]
    n_pages = sum(pages_needed) + 3
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    k_pages = torch.zeros(n_pages, nkv, page_size, dk, dtype=dtype, device=DEV)
    v_pages = k_pages if latent else torch.zeros(n_pages, nkv, page_size, dv, dtype=dtype, device=DEV)
    table = torch.zeros(len(entries), max(pages_needed), dtype=torch.int32)
    for e, t in enumerate(total):
        for p in range(pages_needed[e]):
            page = order.pop()
            table[e, p] = page
            lo, hi = p * page_size, min((p + 1) * page_size, t)
            k_pages[page, :, :hi - lo] = ks[e][lo:hi].transpose(0, 1)
            if not latent:
                v_pages[page, :, :hi - lo] = vs[e][lo:hi].transpose(0, 1)
    q_lens, starts = [n for _, n in entries], [s for s, _ in entries]
    n_tokens = sum(q_lens)
    q_rows = torch.cat(qs).reshape(n_tokens, nq * dk).contiguous()
    ctx = SimpleNamespace(dtype=dtype, token_seq=i32(np.repeat(np.arange(len(entries)), q_lens)), cu_q=i32(np.concatenate([[0], np.cumsum(q_lens)])),
                          q_start_pos=i32(starts), n_seqs=len(entries), n_tokens=n_tokens, max_kv_len=max(total), max_q_len=max(q_lens))
    plan = {k: (i32(v) if len(v) else None)
            for k, v in attention_ops.plan_biased(HostStep(q_lens, starts, n_tokens, len(entries)), group, window or 0, 0).items()}
    kv = KVStep(k_pages, v_pages, None, table.to(DEV), page_size)
    out = attention_ops.attend_biased(ctx, plan, q_rows, kv, nq, nkv, dk, dv, window, 0, scale, None, None, sink, v_row=dk if latent else 0)
    ref = torch.zeros(n_tokens, nq, dv, dtype=torch.float64, device=DEV)
    first = np.concatenate([[0], np.cumsum(q_lens)])
    for e, (s, n) in enumerate(entries):
        i = torch.arange(s, s + n, device=DEV)[:, None]
        j = torch.arange(s + n, device=DEV)[None, :]
        see = (j <= i) & ((i - j) < window if window else torch.ones_like(j <= i))
        for h in range(nq):
            sc = (qs[e][:, h].double() @ ks[e][:, h // group].double().T) * scale
            sc = torch.where(see, sc, torch.tensor(-float("inf"), dtype=torch.float64, device=DEV))
            weights = torch.exp(sc - sc.max(dim=1, keepdim=True).values)
            denom = weights.sum(dim=1, keepdim=True)
            if sink is not None:
                denom = denom + torch.exp(sink[h].double() - sc.max(dim=1, keepdim=True).values)
            ref[first[e]:first[e + 1], h] = (weights / denom) @ vs[e][:, h // group].double()
    return out.double().reshape(n_tokens, nq, dv), ref


def tolerance(dtype):
    return 2e-5 if dtype == torch.float32 else 3e-2


# (query heads, kv heads, key size, value size, values inside the keys): sizes of the tensor-core kernels and others
SHAPES = [(6, 2, 64, 32, False), (4, 4, 32, 64, False), (4, 1, 64, 32, True), (3, 1, 48, 40, True), (20, 1, 128, 64, True), (6, 3, 80, 16, False),
          (4, 1, 80, 64, True), (16, 1, 192, 128, True), (3, 1, 48, 32, True), (5, 1, 160, 128, True), (3, 1, 96, 64, True)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,dk,dv,latent", SHAPES)
def test_attention_edges_of_a_window_with_a_sink(dtype, nq, nkv, dk, dv, latent):
    """Window 40, pages of 16, learned sinks between -2 and 3.  Peaked scores on the key just inside the
    window (i - 39), just outside (i - 40: must not count) and on the query's own key, for tokens of a run
    that starts in the middle of a page and for single tokens."""
    sink = torch.linspace(-2.0, 3.0, nq, device=DEV)
    entries = [(70, 50), (131, 1), (0, 45), (39, 1), (40, 1)]
    peaks = [(0, 10, 0, 80 - 39, 9.0), (0, 11, 1, 81 - 40, 9.0), (0, 49, 2, 119, 9.0), (1, 0, 0, 131 - 39, 9.0), (1, 0, 1, 131 - 40, 9.0),
             (2, 44, 0, 5, 9.0), (2, 44, 1, 4, 9.0), (2, 3, 2, 0, 9.0), (3, 0, 0, 0, 9.0), (4, 0, 0, 0, 9.0), (4, 0, 1, 1, 9.0)]
    got, want = sink_attention_case(dtype, nq, nkv, dk, dv, 16, 40, sink, latent, entries, 11, peaks)
    assert (got - want).abs().max() < tolerance(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,dk,dv,latent", SHAPES)
@pytest.mark.parametrize("page_size", [8, 64])
def test_attention_far_key_among_hundreds_and_a_sink_of_zero(dtype, nq, nkv, dk, dv, latent, page_size):
    """No window: key 3 of 700 carries the weight of a decoded token's head and of a run's token; the
    sink's score is 0 (one is added to the denominator), which halves an output whose scores are near 0."""
    sink = torch.zeros(nq, device=DEV)
    entries = [(699, 1), (500, 130), (0, 1), (300, 1)]
    peaks = [(0, 0, 0, 3, 12.0), (0, 0, nq - 1, 698, 12.0), (1, 129, 1, 3, 12.0), (1, 0, 0, 499, 12.0), (3, 0, 1, 15, 12.0)]
    got, want = sink_attention_case(dtype, nq, nkv, dk, dv, page_size, None, sink, latent, entries, 12, peaks)
    assert (got - want).abs().max() < tolerance(dtype)
    none, _ = sink_attention_case(dtype, nq, nkv, dk, dv, page_size, None, None, latent, entries, 12, peaks)
    assert (none - want).abs().max() > 0.05                  # without the sink the outputs are others


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_large_sink_takes_the_weight(dtype):
    sink = torch.tensor([30.0, -30.0, 0.0, 5.0], device=DEV)
    got, want = sink_attention_case(dtype, 4, 2, 64, 64, 16, 20, sink, False, [(25, 9), (60, 1)], 13, [])
    assert (got - want).abs().max() < tolerance(dtype)
    assert got[:, 0].abs().max() < 1e-6 and got[:, 1].abs().max() > 0.05


# ---- retention ----------------------------------------------------------------------------------------------


def retention_reference(x, heads, dim, vdim, decay, freqs, positions, eps):
    """One request's whole sequence in float64: rows of q | k | v | g."""
    n = x.shape[0]
    x = x.double().cpu().numpy()
    q, k = x[:, :heads * dim].reshape(n, heads, dim), x[:, heads * dim:2 * heads * dim].reshape(n, heads, dim)
    v = x[:, 2 * heads * dim:2 * heads * dim + heads * vdim].reshape(n, heads, vdim)
    gate = x[:, 2 * heads * dim + heads * vdim:]
    q, k = plain.rotate(q, positions, freqs, 1.0, "half"), plain.rotate(k, positions, freqs, 1.0, "half") * dim ** -0.5
    out = np.zeros((n, heads, vdim))
    for h in range(heads):
        S = np.zeros((dim, vdim))
        for t in range(n):
            S = decay[h] * S + np.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return plain.rms_unit(out, eps).reshape(n, heads * vdim) * plain.silu(gate)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,vdim,dims", [(3, 16, 24, 8), (2, 64, 32, 64), (5, 12, 20, 12), (2, 128, 128, 0), (1, 40, 8, 20), (2, 10, 14, 4),
                                                  (1, 256, 256, 64)])
def test_retention_in_portions_with_state(dtype, heads, dim, vdim, dims):
    """Two requests of unequal length in four steps (portions of 1, 2 and many tokens, the second request
    absent from a step), in slots 2 and 0 of three; then a third request in the slot the second one
    left, cleared as the cache manager clears it.  The state carries S; the result is the whole sequence's."""
    g = torch.Generator(device=DEV).manual_seed(4)
    decay = [1.0, 0.5, 0.96875, 0.99, 0.9][:heads]
    freqs, _ = rotary_frequencies(dims, 100.0, None)
    inv_freq = torch.tensor(freqs, dtype=torch.float32, device=DEV)
    width = 2 * heads * dim + 2 * heads * vdim
    lens = {"a": 203, "b": 9, "c": 70}
    x = {k: torch.randn(n, width, generator=g, device=DEV).to(dtype) for k, n in lens.items()}
    want = {k: retention_reference(x[k], heads, dim, vdim, decay, freqs, np.arange(lens[k]), 1e-5) for k in lens}
    state = torch.zeros(3, heads, dim, vdim, device=DEV)
    slot = {"a": 2, "b": 0, "c": 0}
    done = {k: 0 for k in lens}
    got = {k: [] for k in lens}
    for step in ({"a": 1, "b": 2}, {"a": 2}, {"a": 130, "b": 7}, {"c": 69, "a": 70}, {"c": 1}):
        names = list(step)
        if "c" in names and done["c"] == 0:
            state[0].zero_()                               # the slot is handed out again
        rows = torch.cat([x[k][done[k]:done[k] + step[k]] for k in names])
        positions = i32(np.concatenate([np.arange(done[k], done[k] + step[k]) for k in names]))
        cu = i32(np.concatenate([[0], np.cumsum([step[k] for k in names])]))
        slots = i32([slot[k] for k in names])
        angles = kernels.rotary_angles(positions, inv_freq, 1.0) if dims else None
        out = torch.empty(rows.shape[0], heads * vdim, dtype=dtype, device=DEV)
        chunks, runs, short = kernels.plan_retention([step[k] for k in names])       # the run of 130 tokens goes in three chunks, 69 and 70 in two
        kernels.retention(rows, 0, heads * dim, 2 * heads * dim, 2 * heads * dim + heads * vdim, angles, "halves",
                          torch.tensor(decay, dtype=torch.float32, device=DEV), state, cu, slots, out, len(names), max(step.values()),
                          heads, dim, vdim, dim ** -0.5, 1e-5, i32(chunks) if chunks else None, i32(runs) if runs else None, scan_too=short or not chunks)
        at = 0
        for k in names:
            got[k].append(out[at:at + step[k]])
            at += step[k]
            done[k] += step[k]
    assert state[1].abs().max() == 0                                   # nobody's slot stays untouched
    for k in lens:
        err = np.abs(torch.cat(got[k]).double().cpu().numpy() - want[k]).max()
        assert err < (2e-4 if dtype == torch.float32 else 6e-2), (k, err)


# ---- the dense clamped gated feed-forward -----------------------------------------------------------------------


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [3, 8, 40, 300])
@pytest.mark.parametrize("hidden,inter", [(128, 96), (256, 200), (96, 44)])
def test_clamped_glu_feed_forward(dtype, rows, hidden, inter):
    """Steps of up to 8 rows (the unit in the weight-streaming product's epilogue), of some dozens (a kernel of
    its own behind the library's product, on the paired layout) and of hundreds (the tcgen05 product's epilogue);
    a width that has no paired layout (44) takes the plain layout everywhere."""
    from qwen25vl_lite.parts.feed_forward import ClampedGLU

    g = torch.Generator(device=DEV).manual_seed(5)
    rnd = lambda *shape, scale=1.0: torch.randn(*shape, generator=g, device=DEV) * scale
    tensors = {"gate": rnd(inter, hidden, scale=0.2), "up": rnd(inter, hidden, scale=0.2), "down": rnd(hidden, inter, scale=0.2)}
    tensors = {k: v.to(dtype).float() for k, v in tensors.items()}       # what bfloat16 can hold, in both runs
    part = ClampedGLU(hidden, inter, 1.25, 1.702)
    part.load(tensors, DEV, dtype)
    h = rnd(rows, hidden).to(dtype)
    out = part.forward(SimpleNamespace(dtype=dtype), h)
    x, w = h.double(), {k: v.double() for k, v in tensors.items()}
    gate, up = (x @ w["gate"].T).clamp(max=1.25), (x @ w["up"].T).clamp(-1.25, 1.25)
    want = (gate * torch.sigmoid(1.702 * gate) * (up + 1)) @ w["down"].T
    assert (gate == 1.25).any() and (up == -1.25).any()                 # the clamps were reached
    err = (out.double() - want).abs().max()
    assert err < (2e-5 if dtype == torch.float32 else 0.03 * float(want.abs().max())), float(err)
