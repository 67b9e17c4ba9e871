"""Vepivik on the GPU against the plain implementation: every mechanism's kernel alone, then whole models cut into
steps in every way, then generation through the entry point.

Kernel tests build their own index arrays and pages (handed out shuffled) and compare with the functions of
``plain_vepivik`` or with sums written out here, in float64.  Where random numbers would hide a fault (a window that
is one position off, a far key among hundreds) one key is made to stand out.  Model tests make small model
folders of four configurations that differ in every size and option and replay requests whole, with a decoded
tail, in portions down to two tokens, and mixed with few pages and slots.
"""

import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_vepivik as plain
import traces
from vepivik_models import vepivik_dir

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def i32(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


def shuffled_pages(n_tokens, page, seed, spare=3):
    """(table int32 [1, pages], page id of every token, slot in its page) for one request whose pages lie anywhere."""
    pages = -(-n_tokens // page)
    perm = torch.randperm(pages + spare, generator=torch.Generator().manual_seed(seed))[:pages]
    return perm.to(torch.int32).reshape(1, -1).to(DEV), [int(perm[t // page]) for t in range(n_tokens)], [t % page for t in range(n_tokens)]


# ---- rotation, the latent's norm and its place in the pages ---------------------------------------------------

@pytest.mark.parametrize("dtype, heads, d, r, p, dims, interleaved, scaling", [
    (torch.float32, 3, 5, 14, 8, 8, True, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 2.0}),
    (torch.float32, 2, 8, 40, 6, 4, True, None),
    (torch.bfloat16, 4, 16, 64, 32, 32, True, {"factor": 2.0, "original": 64, "fast": 16.0, "slow": 1.0}),
    (torch.float32, 1, 4, 9, 4, 4, False, None)])
def test_latent_prepare_norms_rotates_and_places_rows(dtype, heads, d, r, p, dims, interleaved, scaling):
    from yalis_b200.ops.latent import latent_prepare
    from yalis_b200.parts.rotary import inverse_frequencies, yarn_frequencies
    g = torch.Generator().manual_seed(r)
    rot = {"dims": dims, "base": 50.0, "scaling": scaling}
    if scaling is None:
        freq, mag = inverse_frequencies(dims, 50.0, None, exact_powers=True), 1.0
    else:
        freq, mag = yarn_frequencies(dims, 50.0, scaling["factor"], scaling["original"], scaling["fast"], scaling["slow"])
    page, start, n = 8, 1000, 21                       # positions 1000..1020: angles that a table of a few hundred would miss
    table, page_of, slot_of = shuffled_pages(start + n, page, seed=1)
    q_off, kv_off = 8, 8 + heads * (d + p) + 3
    src = (torch.randn(n, kv_off + r + p + 2, generator=g) * 2).to(dtype)
    norm_w = 1 + 0.3 * torch.randn(r, generator=g)
    pool = torch.full((table.shape[1] + 3, 1, page, r + p), 7.0, dtype=dtype, device=DEV)
    qc = torch.full((n, heads, r + p), -3.0, device=DEV)
    positions = list(range(start, start + n))
    latent_prepare(src.to(DEV), q_off, kv_off, heads, d, r, p, norm_w.to(DEV), 1e-3, freq.to(DEV), interleaved, mag, qc, pool, table,
                   i32(positions), i32([0] * n))
    x = src.double()
    tol = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    # the angle is a 32-bit product by design: near position 1000 it is known to 6e-5, which values of 2 to 6 carry over
    rot_tol = dict(rtol=2e-5, atol=5e-4) if dtype == torch.float32 else dict(rtol=1e-2, atol=2e-2)
    if interleaved:
        want_q = plain.rotate_pairs(x[:, q_off:q_off + heads * (d + p)].reshape(n, heads, d + p)[..., d:], positions, rot)
        want_k = plain.rotate_pairs(x[:, kv_off + r:kv_off + r + p], positions, rot)
    else:                                               # halves: size i with size i + dims / 2
        def halves(v):
            out = v.clone()
            f, _ = plain.rotary_frequencies(rot)
            for ti, pos in enumerate(positions):
                for i, fi in enumerate(f):
                    c, s = math.cos(pos * fi), math.sin(pos * fi)
                    a, b = v[ti, ..., i].clone(), v[ti, ..., i + dims // 2].clone()
                    out[ti, ..., i], out[ti, ..., i + dims // 2] = a * c - b * s, b * c + a * s
            return out
        want_q = halves(x[:, q_off:q_off + heads * (d + p)].reshape(n, heads, d + p)[..., d:])
        want_k = halves(x[:, kv_off + r:kv_off + r + p])
    torch.testing.assert_close(qc[:, :, r:].double().cpu(), want_q, **rot_tol)
    assert bool((qc[:, :, :r] == -3.0).all())                                   # the other columns are someone else's
    want_c = plain.rms_norm(x[:, kv_off:kv_off + r], norm_w.double(), 1e-3)
    rows = torch.stack([pool[page_of[t], 0, slot_of[t]] for t in positions]).double().cpu()
    torch.testing.assert_close(rows[:, :r], want_c, **tol)
    torch.testing.assert_close(rows[:, r:], want_k, **rot_tol)
    untouched = pool.clone()
    for t in positions:
        untouched[page_of[t], 0, slot_of[t]] = 7.0
    assert bool((untouched == 7.0).all())                                        # nothing else was written
    # a layer that reads another layer's rows writes none
    before = pool.clone()
    latent_prepare(src.to(DEV), q_off, None, heads, d, r, p, None, 1e-3, freq.to(DEV), interleaved, mag, qc, pool, table,
                   i32(positions), i32([0] * n))
    assert torch.equal(before, pool)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_project_with_and_without_a_gate(dtype):
    from yalis_b200.ops.latent import head_project
    g = torch.Generator().manual_seed(3)
    n, h, k, o = 9, 3, 37, 11
    w = torch.randn(h, o, k, generator=g).to(dtype)
    wide = torch.randn(n, 4 + h * (k + 5), generator=g).to(dtype)                 # heads with 5 more columns each
    x = wide[:, 4:].unflatten(1, (h, k + 5))[:, :, :k]
    want = torch.einsum("hok,nhk->nho", w.double(), x.double())
    out = torch.zeros(n, h, o + 2, device=DEV)
    head_project(x.to(DEV), w.to(DEV), out[:, :, :o], req_of_token=i32([0] * 4 + [-1] + [1] * 4))
    want_rows = want.clone()
    want_rows[4] = 0                                                               # a row of no request is skipped
    torch.testing.assert_close(out[:, :, :o].double().cpu(), want_rows, rtol=1e-5, atol=1e-5)
    gate = torch.randn(n, h * o, generator=g).to(dtype)
    xf = torch.randn(n, h, k, generator=g)
    y = torch.zeros(n, h * o + 8, dtype=dtype, device=DEV)
    head_project(xf.to(DEV), w.to(DEV), y[:, 8:].unflatten(1, (h, o)), gate=gate.to(DEV))
    want = torch.einsum("hok,nhk->nho", w.double(), xf.double()).reshape(n, h * o) * torch.sigmoid(gate.double())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(y[:, 8:].double().cpu(), want, rtol=tol, atol=tol)


# ---- attention over rows: windows, page borders, far keys -------------------------------------------------------------

def plain_rows_attention(qc, rows, r, scale, window, pos):
    lo = max(0, pos - window + 1) if window else 0
    s = (rows[lo:pos + 1] @ qc) * scale
    return plain.softmax_rows(s[None])[0] @ rows[lo:pos + 1, :r]


@pytest.mark.parametrize("dtype, r, p, page, window", [(torch.float32, 24, 8, 16, 37), (torch.bfloat16, 64, 32, 8, 64),
                                                       (torch.float32, 14, 4, 16, 1), (torch.float32, 20, 2, 64, None),
                                                       (torch.float32, 512, 64, 16, 100)])
def test_latent_attention_sees_exactly_its_window(dtype, r, p, page, window):
    """One row is made to stand out; queries whose window just holds it answer with it, the next ones do not."""
    from yalis_b200.ops.latent import latent_attention_exact
    g = torch.Generator().manual_seed(r + p)
    T, heads = 400, 3
    W = window or T
    star = 15 if page == 16 else (63 if page == 64 else 7)                       # the last place of a page
    rows = torch.randn(T, r + p, generator=g) * 0.3
    u = torch.nn.functional.normalize(torch.randn(r + p, generator=g), dim=0)
    rows[star] = 6.0 * u
    rows = rows.to(dtype)
    table, page_of, slot_of = shuffled_pages(T, page, seed=5)
    pool = torch.zeros(table.shape[1] + 3, 1, page, r + p, dtype=dtype, device=DEV)
    pool.fill_(float("nan"))                                                      # what no request holds must not be read
    for t in range(T):
        pool[page_of[t], 0, slot_of[t]] = rows[t].to(DEV)
    edge = star + W - 1                                                           # the last position that sees the row
    ask = sorted({star, min(edge - 1, T - 1), min(edge, T - 1), min(edge + 1, T - 1), min(edge + 2, T - 1), T - 1, 0})
    qc = torch.randn(len(ask), heads, r + p, generator=g) * 0.3
    qc[:, 1] = 4.0 * u                                                            # head 1 asks for the planted row
    scale = 1.0
    for name, groups in (("together", [ask]), ("one by one", [[a] for a in ask])):  # a prompt's portion, decoded tokens
        got = {}
        at = 0
        for grp in groups:
            out = latent_attention_exact(qc[at:at + len(grp)].contiguous().to(DEV), pool, i32(grp), i32([0] * len(grp)), table, r, scale, window)
            for j, a in enumerate(grp):
                got[a] = out[j].double().cpu()
            at += len(grp)
        for j, a in enumerate(ask):
            for h in range(heads):
                want = plain_rows_attention(qc[j, h].double(), rows.double(), r, scale, window, a)
                tol = 2e-5 if dtype == torch.float32 else 2e-2
                torch.testing.assert_close(got[a][h], want, rtol=tol, atol=tol, msg=lambda m: f"{name} position {a} head {h}: {m}")
            hit = float(torch.dot(got[a][1], rows[star, :r].double()) / rows[star, :r].double().norm() ** 2)
            if star <= a <= edge:
                assert hit > 0.9, (name, a, hit)              # 24 in the exponent: the planted row takes the weight
            else:
                assert hit < 0.5, (name, a, hit)


@pytest.mark.parametrize("r, p, page, window, heads", [(64, 32, 8, 64, 3), (96, 32, 16, 37, 3), (128, 0, 64, None, 2),
                                                      (256, 64, 16, 100, 16), (512, 64, 32, 150, 5), (384, 48, 16, 1, 8)])
def test_latent_attention_on_the_tensor_cores(r, p, page, window, heads):
    """The same sums by the tensor-core form: two requests in one step (a portion of 45 tokens behind 250 cached ones
    beside a single token), the planted row at the window's edge of some of the portion's tokens; queries given in
    float32 and, head-major, in bfloat16; results taken in both forms."""
    from yalis_b200.ops.latent import latent_attention_mma
    g = torch.Generator().manual_seed(r + p)
    W = window or 10 ** 6
    lens, new = [295, 130], [45, 1]
    first = lens[0] - new[0]                                                      # position of the portion's first token
    star = first + 20 - (W - 1) if window and first + 20 - (W - 1) >= 0 else 7    # seen by the portion's first 21 tokens only
    u = torch.nn.functional.normalize(torch.randn(r + p, generator=g), dim=0)
    rows, tables, pages_used = [], [], 0
    pool = torch.full((sum(-(-l // page) for l in lens) + 2, 1, page, r + p), float("nan"), dtype=torch.bfloat16, device=DEV)
    width = max(-(-l // page) for l in lens)
    table = torch.full((2, width), -1, dtype=torch.int32)
    perm = torch.randperm(pool.shape[0], generator=g).tolist()
    for i, l in enumerate(lens):
        rw = torch.randn(l, r + p, generator=g) * 0.3
        if i == 0:
            rw[star] = 6.0 * u
        rw = rw.to(torch.bfloat16)
        rows.append(rw)
        for t in range(l):
            if t % page == 0:
                table[i, t // page] = perm.pop()
            pool[int(table[i, t // page]), 0, t % page] = rw[t].to(DEV)
    positions = list(range(first, lens[0])) + [lens[1] - 1]
    n = len(positions)
    qc = (torch.randn(n, heads, r + p, generator=g) * 0.3)
    qc[:, 1] = 4.0 * u
    qc = qc.to(torch.bfloat16).float()                                            # what both forms of the queries can hold
    q_start, table = i32([0, new[0], n]), table.to(DEV)
    out32 = torch.zeros(n, heads, r, device=DEV)
    qd = qc.to(DEV)
    req = i32([0] * new[0] + [1])
    latent_attention_mma(qd[:, :, :r], qd[:, :, r:], out32, pool, i32(positions), q_start, req, table, 2, max(new), 0.5, window)
    q_lat = qc[:, :, :r].to(torch.bfloat16).transpose(0, 1).contiguous().to(DEV)            # [H, N, r]
    out16 = torch.zeros(heads, n, r, dtype=torch.bfloat16, device=DEV)
    latent_attention_mma(q_lat.transpose(0, 1), qd[:, :, r:].contiguous(), out16.transpose(0, 1), pool, i32(positions), q_start,
                         req, table, 2, max(new), 0.5, window)
    # single tokens of both requests (the last of each), their rows dealt to 1, 3 and 16 blocks
    last = [new[0] - 1, n - 1]
    for splits in (1, 3, 16):
        one = torch.zeros(2, heads, r, device=DEV)
        latent_attention_mma(qd[last][:, :, :r], qd[last][:, :, r:], one, pool, i32([positions[j] for j in last]), i32([0, 1, 2]),
                             i32([0, 1]), table, 2, 1, 0.5, window, n_splits=splits)
        torch.testing.assert_close(one, out32[last], rtol=1e-4, atol=1e-4, msg=lambda m: f"{splits} splits: {m}")
    for j, a in enumerate(positions):
        which = 0 if j < new[0] else 1
        for h in range(heads):
            want = plain_rows_attention(qc[j, h].double(), rows[which].double(), r, 0.5, window, a)
            torch.testing.assert_close(out32[j, h].double().cpu(), want, rtol=3e-3, atol=3e-3, msg=lambda m: f"position {a} head {h}: {m}")
            torch.testing.assert_close(out16[h, j].double().cpu(), want, rtol=2e-2, atol=2e-2)
        if which == 0 and heads > 1:
            hit = float(torch.dot(out32[j, 1].double().cpu(), rows[0][star, :r].double()) / rows[0][star, :r].double().norm() ** 2)
            assert (hit > 0.9) == (star <= a <= star + W - 1), (a, hit)



@pytest.mark.parametrize("dtype, hs, vd, page, window", [(torch.float32, 12, 20, 16, 9), (torch.bfloat16, 56, 24, 16, 45),
                                                         (torch.float32, 10, 6, 8, 5), (torch.bfloat16, 64, 64, 64, 64)])
def test_windowed_attention_without_positions_sees_exactly_its_window(dtype, hs, vd, page, window):
    from yalis_b200.ops.attention import paged_attention_generic
    g = torch.Generator().manual_seed(hs)
    T, H, G = 300, 4, 2
    star = 2 * page - 1
    k = torch.randn(T, G, hs, generator=g) * 0.3
    v = torch.randn(T, G, vd, generator=g)
    u = torch.nn.functional.normalize(torch.randn(hs, generator=g), dim=0)
    k[star, 1] = 6.0 * u
    k, v = k.to(dtype), v.to(dtype)
    table, page_of, slot_of = shuffled_pages(T, page, seed=2)
    k_pool = torch.zeros(table.shape[1] + 3, G, page, hs, dtype=dtype, device=DEV)
    v_pool = torch.zeros(table.shape[1] + 3, G, page, vd, dtype=dtype, device=DEV)
    for t in range(T):
        k_pool[page_of[t], :, slot_of[t]] = k[t].to(DEV)
        v_pool[page_of[t], :, slot_of[t]] = v[t].to(DEV)
    edge = star + window - 1
    ask = [star, edge - 1, edge, edge + 1, T - 1]
    q = (torch.randn(len(ask), H, hs, generator=g) * 0.3)
    q[:, 2] = 4.0 * u                                                             # head 2 uses key head 1
    q = q.to(dtype)
    out = paged_attention_generic(q.reshape(len(ask), H * hs).to(DEV), k_pool, v_pool, i32(ask), i32([0] * len(ask)), table, H, G, hs,
                                  scale=1.0, window=window, v_head_dim=vd).double().cpu().reshape(len(ask), H, vd)
    group = [h // (H // G) for h in range(H)]
    for j, a in enumerate(ask):
        lo = max(0, a - window + 1)
        for h in range(H):
            s = k[lo:a + 1, group[h]].double() @ q[j, h].double()
            want = plain.softmax_rows(s[None])[0] @ v[lo:a + 1, group[h]].double()
            tol = 2e-5 if dtype == torch.float32 else 2e-2
            torch.testing.assert_close(out[j, h], want, rtol=tol, atol=tol)
        near = float((out[j, 2] - v[star, 1].double()).abs().max())
        assert (near < 0.05) == (star <= a <= edge), (a, near)


# ---- the routed feed-forward ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("n, experts, top", [(50, 8, 3), (7, 5, 5), (33, 64, 6), (4, 3, 1), (20, 130, 8)])
def test_route_topk_against_the_plain_router(n, experts, top):
    from yalis_b200.ops.experts import route_topk
    g = torch.Generator().manual_seed(experts)
    logits = torch.randn(n, experts, generator=g) * 3
    logits[1, :] = 0.0                                            # all equal: ties go to the smaller index
    ids, w = route_topk(logits.to(DEV), top, 1e-20, i32([0] * (n - 1) + [-1]))
    s = plain.softmax_rows(logits.double())
    for t in range(n - 1):
        order = sorted(range(experts), key=lambda e: (-float(s[t, e]), e))[:top]
        assert ids[t].tolist() == order, t
        want = s[t, order] / (s[t, order].sum() + 1e-20)
        torch.testing.assert_close(w[t].double().cpu(), want, rtol=1e-5, atol=1e-7)
    assert ids[n - 1].tolist() == [-1] * top                      # a row of no request chooses nothing


def ff_tensors(hidden, experts, inner, shared, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    t = {"router": (torch.randn(experts, hidden, generator=g) * 3 / hidden ** 0.5).to(torch.bfloat16)}
    for e in range(experts):
        t[f"e{e}.up"] = (torch.randn(inner, hidden, generator=g) / hidden ** 0.5).to(torch.bfloat16)
        t[f"e{e}.down"] = (torch.randn(hidden, inner, generator=g) / inner ** 0.5).to(torch.bfloat16)
    if shared:
        t["shared.up"] = (torch.randn(shared, hidden, generator=g) / hidden ** 0.5).to(torch.bfloat16)
        t["shared.down"] = (torch.randn(hidden, shared, generator=g) / shared ** 0.5).to(torch.bfloat16)
    return t


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n, hidden, experts, top, inner, shared", [
    (5, 64, 4, 2, 24, 40), (70, 36, 5, 3, 18, None), (900, 128, 4, 2, 64, 64), (300, 128, 16, 4, 40, 8), (1, 40, 2, 2, 7, 3)])
def test_routed_experts_against_the_plain_mixture(dtype, n, hidden, experts, top, inner, shared):
    """The part alone: few tokens, rows off 16-byte boundaries, enough tokens an expert for the large row tile,
    inner sizes that are no multiple of a tile, every expert chosen."""
    from yalis_b200.config.spec import PartSpec
    from yalis_b200.parts.base import make_part
    t = ff_tensors(hidden, experts, inner, shared, seed=n, dtype=dtype)
    part = make_part("feed_forward", PartSpec("routed_experts", {"hidden_size": hidden, "experts": experts, "top": top,
                                                                 "expert_size": inner, "activation": "relu2", "shared_size": shared}))
    local = {"router": t["router"].float().to(DEV)}
    for e in range(experts):
        local[f"expert_{e}_up"], local[f"expert_{e}_down"] = t[f"e{e}.up"].to(dtype).to(DEV), t[f"e{e}.down"].to(dtype).to(DEV)
    if shared:
        local["shared_up"], local["shared_down"] = t["shared.up"].to(dtype).to(DEV), t["shared.down"].to(dtype).to(DEV)
    part.load(local)
    x = torch.randn(n, hidden, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    got = part.forward(x.to(dtype).to(DEV), None).double().cpu()
    mlp = {"router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    want = plain.mixture_of_experts(x.double(), {"p." + k: v.double() for k, v in t.items()}, "p.", mlp)
    if dtype == torch.float32:
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)
    else:
        # bfloat16 rounds the inner activations and the experts' results; a token whose router scores are nearly equal
        # may also choose another expert than float64 does, so a few rows may differ
        err = (got - want).abs().max(dim=1).values / want.abs().max()
        assert float(err.median()) < 2e-2 and float((err > 4e-2).float().mean()) <= 0.03, float(err.max())


@pytest.mark.parametrize("n, hidden, experts, top, inner, shared", [(8, 128, 16, 2, 64, 32), (70, 64, 4, 2, 72, None), (600, 128, 4, 2, 200, 64),
                                                                  (2500, 256, 8, 2, 136, None), (40, 64, 2, 2, 8, None)])
def test_the_two_tensor_core_forms_of_the_experts_products_agree(n, hidden, experts, top, inner, shared, monkeypatch):
    """tcgen05 with TMA-streamed operands (every row tile from 16 to 256, experts with more rows than a tile, inner sizes
    that end inside a 128-row box of weights) against the mma.sync form and the plain mixture; no wait runs out."""
    from yalis_b200.config.spec import PartSpec
    from yalis_b200.ops import _lib
    from yalis_b200.parts.base import make_part
    t = ff_tensors(hidden, experts, inner, shared, seed=n, dtype=torch.bfloat16)
    part = make_part("feed_forward", PartSpec("routed_experts", {"hidden_size": hidden, "experts": experts, "top": top,
                                                                 "expert_size": inner, "activation": "relu2", "shared_size": shared}))
    local = {"router": t["router"].float().to(DEV)}
    for e in range(experts):
        local[f"expert_{e}_up"], local[f"expert_{e}_down"] = t[f"e{e}.up"].to(DEV), t[f"e{e}.down"].to(DEV)
    if shared:
        local["shared_up"], local["shared_down"] = t["shared.up"].to(DEV), t["shared.down"].to(DEV)
    part.load(local)
    x = torch.randn(n, hidden, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(DEV)
    monkeypatch.delenv("YALIS_B200_NO_GROUPED_TCGEN05", raising=False)
    streamed = part.forward(x, None)
    assert torch.equal(streamed, part.forward(x, None))
    monkeypatch.setenv("YALIS_B200_NO_GROUPED_TCGEN05", "1")
    other = part.forward(x, None)
    assert int(_lib.error_word(x.device).item()) == 0
    # the same routing, float32 sums of the same bfloat16 products in another order, one rounding: a few last bits apart
    diff = (streamed.float() - other.float()).abs().max(dim=1).values / other.float().abs().max()
    assert float(diff.max()) < 2e-2 and float((diff > 4e-3).float().mean()) < 0.02, float(diff.max())
    mlp = {"router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    want = plain.mixture_of_experts(x.double().cpu(), {"p." + k: v.double() for k, v in t.items()}, "p.", mlp)
    err = (streamed.double().cpu() - want).abs().max(dim=1).values / want.abs().max()
    assert float(err.median()) < 2e-2 and float((err > 4e-2).float().mean()) <= 0.03, float(err.max())


def test_the_order_of_tokens_inside_an_expert_leaves_no_trace():
    """The grouping uses atomics; the results must have the same bits every time, and a token's result must not depend
    on what else is in the batch."""
    from yalis_b200.config.spec import PartSpec
    from yalis_b200.parts.base import make_part
    for dtype in (torch.float32, torch.bfloat16):
        t = ff_tensors(64, 8, 32, 16, seed=4, dtype=dtype)
        part = make_part("feed_forward", PartSpec("routed_experts", {"hidden_size": 64, "experts": 8, "top": 2, "expert_size": 32,
                                                                     "activation": "relu2", "shared_size": 16}))
        local = {"router": t["router"].float().to(DEV), "shared_up": t["shared.up"].to(dtype).to(DEV), "shared_down": t["shared.down"].to(dtype).to(DEV)}
        for e in range(8):
            local[f"expert_{e}_up"], local[f"expert_{e}_down"] = t[f"e{e}.up"].to(dtype).to(DEV), t[f"e{e}.down"].to(dtype).to(DEV)
        part.load(local)
        x = torch.randn(200, 64, generator=torch.Generator().manual_seed(2)).to(dtype).to(DEV)
        first = part.forward(x, None)
        for _ in range(3):
            assert torch.equal(first, part.forward(x, None))
        alone = torch.cat([part.forward(x[i:i + 1], None) for i in (0, 57, 199)])
        if dtype == torch.float32:
            assert torch.equal(alone, first[[0, 57, 199]])
        else:           # the shared expert's product goes to another kernel for one token than for 200
            torch.testing.assert_close(alone.float(), first[[0, 57, 199]].float(), rtol=2e-2, atol=2e-2)


# ---- whole models -----------------------------------------------------------------------------------------------------

TOL = {"float32": 1e-4, "bfloat16": 5e-2}       # relative to the largest |logit| of the request
LENGTHS = {"A": [1, 5, 33, 70, 21, 48], "B": [2, 40, 9, 64, 17, 90], "C": [3, 37, 18, 130, 12, 66], "D": [7, 1, 50, 19, 33, 4]}
PAGE = {"A": 16, "B": 8, "C": 64, "D": 16}
_oracle = {}


def requests_for(which):
    cfg, _ = plain.read_folder(vepivik_dir(which))
    g = torch.Generator().manual_seed(ord(which))
    return {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate(LENGTHS[which])}


def oracle(which):
    if which not in _oracle:
        cfg, w = plain.read_folder(vepivik_dir(which))
        _oracle[which] = {rid: plain.forward(cfg, w, t)[0].numpy() for rid, t in requests_for(which).items()}
    return _oracle[which]


def replay(which, dtype, steps, max_tokens, graphs=False):
    from yalis_b200.engine.replay import Replayer
    rep = Replayer(vepivik_dir(which), dtype, max_tokens, page_size=PAGE[which], graphs=graphs)
    out = {}
    for s in steps:
        r = rep.run_step(s)
        if r is not None:
            out[s["step"]] = r
    rep.engine.manager.check()
    for grp in rep.engine.groups:
        assert rep.engine.manager.free_pages(grp.name) == grp.num_pages          # every page came back
    return out, rep


def compare(got, want, tol, what, outliers=0.0):
    assert set(got) == set(want), what
    total = bad = 0
    for rid in want:
        assert got[rid].shape == want[rid].shape, (what, rid)
        scale = np.abs(want[rid]).max()
        err = np.abs(got[rid] - want[rid]).max(axis=1) / scale
        total += len(err)
        bad += int((err > tol).sum())
        if err.max() > tol and not outliers:
            raise AssertionError(f"{what}: request {rid} differs by {err.max():.3e} (tolerance {tol}); first wrong "
                                 f"position {int(np.argmax(err > tol))} of {len(err)}")
    assert bad <= outliers * total, f"{what}: {bad} of {total} positions differ by more than {tol}"


@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_requests_cut_four_ways_agree_with_the_plain_model(which, dtype):
    reqs, want = requests_for(which), oracle(which)
    vocab = plain.read_folder(vepivik_dir(which))[0]["vocab"]
    results = {}
    # bfloat16: a token whose two best router scores are nearly equal may run another expert than the float64 model
    outliers = 0.0 if dtype == "float32" else 0.06
    for name, steps in (("whole", traces.whole(reqs)), ("tail", traces.tail_decoded(reqs, tail=12)),
                        ("portions", traces.portions(reqs, seed=3)), ("mixed", traces.mixed(reqs, seed=5, tail=6))):
        steps = traces.number(steps)
        out, rep = replay(which, dtype, steps, traces.peak_tokens(steps, max(64, PAGE[which])))
        got = traces.collect(steps, out, vocab)
        compare(got, want, TOL[dtype], f"{which} {dtype} {name}", outliers=outliers)
        results[name] = got
    # how a request was cut, what ran beside it and which pages and slots it had leave (nearly) no trace
    for name in ("tail", "portions", "mixed"):
        for rid in want:
            scale = np.abs(want[rid]).max()
            diff = np.abs(results[name][rid] - results["whole"][rid]).max(axis=1) / scale
            if dtype == "float32":
                assert diff.max() < 2e-5, (name, rid)
            else:
                assert np.mean(diff > 5e-2) <= outliers, (name, rid)


@pytest.mark.parametrize("which", ["A", "C"])
def test_steps_replayed_from_recordings_give_the_same(which):
    """Decoded tokens through recorded steps (CUDA graphs): the routing is decided on the device every time."""
    reqs, want = requests_for(which), oracle(which)
    vocab = plain.read_folder(vepivik_dir(which))[0]["vocab"]
    steps = traces.number(traces.tail_decoded(reqs, tail=12))
    launched, _ = replay(which, "float32", steps, traces.peak_tokens(steps, max(64, PAGE[which])))
    recorded, rep = replay(which, "float32", steps, traces.peak_tokens(steps, max(64, PAGE[which])), graphs=True)
    assert rep.steps_replayed > 40
    a, b = traces.collect(steps, launched, vocab), traces.collect(steps, recorded, vocab)
    compare(b, want, TOL["float32"], f"{which} recorded")
    for rid in a:
        assert np.abs(a[rid] - b[rid]).max() / np.abs(a[rid]).max() < 1e-6


def test_the_residual_stream_after_every_layer():
    from yalis_b200.engine.engine import Engine, StepEntry
    d = vepivik_dir("A")
    cfg, w = plain.read_folder(d)
    tokens = requests_for("A")["r2"]
    _, want = plain.forward(cfg, w, tokens)
    eng = Engine(d, dtype="float32", page_size=16, num_pages=8, max_slots=2, max_context=128)
    eng.add_request("x")
    seen = []
    inner = eng.model.forward
    eng.model.forward = lambda ctx, caches: inner(ctx, caches, tap=lambda i, x: seen.append(x.double().cpu()))
    eng.run([StepEntry("x", tokens, [len(tokens) - 1])])
    assert len(seen) == len(want) == 5
    for i, (a, b) in enumerate(zip(seen, want)):
        assert float((a - b).abs().max() / b.abs().max()) < 2e-5, f"layer {i}"


@pytest.mark.parametrize("which, dtype", [("A", "float32"), ("B", "float32"), ("A", "bfloat16")])
def test_long_decoding_keeps_to_the_plain_model(which, dtype):
    """300 tokens one by one after a two-token prompt: every window passes over decoded tokens many times, and the
    pages behind the windows are given back and used again (the pool is far smaller than the sequence)."""
    from yalis_b200.engine.engine import Engine, StepEntry
    d = vepivik_dir(which)
    cfg, w = plain.read_folder(d)
    g = torch.Generator().manual_seed(9)
    tokens = torch.randint(0, cfg["vocab"], (302,), generator=g).tolist()
    want = plain.forward(cfg, w, tokens)[0].numpy()
    eng = Engine(d, dtype=dtype, page_size=8, num_pages=12, max_slots=2, max_context=384)
    eng.add_request("x")
    rows = [eng.run([StepEntry("x", tokens[:2], [0, 1])]).logits.cpu().numpy()]
    for t in tokens[2:]:
        rows.append(eng.run([StepEntry("x", [t], [0])]).logits.cpu().numpy())
    got = np.concatenate(rows)
    eng.check_device_errors()
    err = np.abs(got - want).max(axis=1) / np.abs(want).max()
    if dtype == "float32":
        assert err.max() < 1e-4
    else:
        assert np.mean(err > 5e-2) < 0.06


def test_a_slot_and_its_pages_used_again_start_clean():
    from yalis_b200.engine.engine import Engine, StepEntry
    d = vepivik_dir("C")
    reqs = requests_for("C")
    eng = Engine(d, dtype="float32", page_size=64, num_pages=3, max_slots=1, max_context=192)
    first = None
    for rid in ("r3", "r1", "r3"):
        assert eng.add_request(rid) == 0                       # the only slot, every time
        out = eng.run([StepEntry(rid, reqs[rid], [len(reqs[rid]) - 1])]).logits.cpu().numpy()
        eng.finish_request(rid)
        if rid == "r3":
            if first is None:
                first = out
            else:
                assert np.array_equal(first, out)              # what r1 left in slot and pages does not show


@pytest.mark.parametrize("which", ["A", "B"])
def test_greedy_generation_through_the_entry_point(which):
    from yalis_b200 import InferenceConfig, LLMEngine, ModelConfig
    d = vepivik_dir(which)
    cfg, w = plain.read_folder(d)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (3, 19, 40, 7, 26)]
    engine = LLMEngine(ModelConfig(model_name=f"vepivik-tiny-{which}", model_path=d, precision="fp32"),
                       InferenceConfig(max_batch_size=3, max_length_of_generated_sequences=64, temperature=0.0, top_p=0.0,
                                       page_size=PAGE[which]))
    tokens, metrics = engine.generate(prompts, tokens_to_generate=10)[:2]
    for p, row in zip(prompts, tokens.cpu().tolist()):
        assert row == plain.greedy(cfg, w, p, 10)


def test_the_replay_program_runs_a_vepivik_folder(tmp_path):
    reqs = {k: v for k, v in requests_for("B").items() if k in ("r1", "r2")}
    steps = traces.number(traces.portions(reqs, seed=1))
    out_dir = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", vepivik_dir("B"), "--dtype", "float32",
                           "--out", str(out_dir), "--max-tokens", str(traces.peak_tokens(steps))],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    vocab = plain.read_folder(vepivik_dir("B"))[0]["vocab"]
    outputs = {s["step"]: np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4") for s in steps}
    compare(traces.collect(steps, outputs, vocab), {k: oracle("B")[k] for k in reqs}, TOL["float32"], "program")
