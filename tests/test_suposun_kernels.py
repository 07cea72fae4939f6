"""Suposun's kernels, each alone against the plain functions on inputs of its own: the preparation of queries and keys
(norms, pairings, scaled rotation, values that are the keys), attention with a cap, kept first keys and sinks at every edge,
the bigram embedding over several steps, the router by sigmoid scores, the bounded gate and the GELU gate."""
import math
import os
import types

import pytest
import torch

import plain_suposun as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(t, dtype=None):
    return t.to(dtype if dtype is not None else (torch.float32 if t.is_floating_point() else t.dtype)).to(DEV).contiguous()


def close(got, want, tol, what):
    got, want = got.double().cpu(), want.double()
    assert torch.isfinite(got).all(), f"{what}: not finite"
    err = float((got - want).abs().max() / max(1e-9, float(want.abs().max())))
    assert err < tol, f"{what}: error {err:.3e} of the largest value"


class PagedKV:
    """A paged cache with a permuted block table and NaN in every place that nothing wrote."""

    def __init__(self, n_slots, max_len, G, dk, dv, dtype):
        self.max_blocks = (max_len + 63) // 64
        nb = n_slots * self.max_blocks + 3
        self.k = torch.full((nb, G, 64, dk), float("nan"), dtype=dtype, device=DEV)
        self.v = torch.full((nb, G, 64, dv), float("nan"), dtype=dtype, device=DEV)
        perm = torch.randperm(nb, generator=torch.Generator().manual_seed(1))[:n_slots * self.max_blocks]
        self.table = dev(perm.view(n_slots, self.max_blocks), torch.int32)

    def rows(self, slot, n, which):
        t = self.table[slot].cpu()
        src = self.k if which == "k" else self.v
        return torch.stack([src[int(t[p // 64]), :, p % 64].float().cpu() for p in range(n)])          # [n, G, size]


# (32-bit: an angle of some thousand radians is itself rounded to a few 1e-4, which is what the bound allows for)
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 6e-3)])
@pytest.mark.parametrize("H,G,dk,norm,pairing,rot,scaling,own_values", [
    (4, 1, 16, "head", "interleaved", 8, (4.0, 64, 8.0, 2.0), False), (3, 3, 24, "all", "half", 24, None, True),
    (5, 1, 12, "head", "interleaved", 6, (2.0, 32, 4.0, 1.0), False), (2, 2, 64, "all", "half", 16, None, True),
    (6, 2, 8, None, "interleaved", 8, None, False), (40, 8, 8, "all", "half", 4, None, True), (1, 1, 32, "head", "half", 0, None, False)])
def test_queries_and_keys_prepared(H, G, dk, norm, pairing, rot, scaling, own_values, dtype, tol):
    """Tokens of three sequences at positions across block borders (one far out, where the scaled frequencies matter): the
    queries' rows and what the cache holds, against norm and rotation written out; then the same rows for a layer that
    writes no cache, which must leave the cache alone and never read key columns (they are NaN)."""
    from vlrf_b200.csrc import ops
    g = torch.Generator().manual_seed(H * 100 + dk)
    dv = 20 if own_values else dk
    positions = [0, 1, 2, 63, 64, 65, 1000, 1001, 4000]
    slot_of = [0, 0, 0, 1, 1, 1, 2, 2, 1]
    T, eps = len(positions), 1e-5
    q, k, v = (torch.randn(T, n, generator=g) * 2.0 for n in (H * dk, G * dk, G * dv))
    wq = 1.0 + 0.3 * torch.randn(dk if norm == "head" else H * dk, generator=g)
    wk = 1.0 + 0.3 * torch.randn(dk if norm == "head" else G * dk, generator=g)
    cols = [q, k] + ([v] if own_values else [])
    proj = torch.cat(cols, dim=1)
    wide = torch.full((T, proj.shape[1] + 4), float("nan"))
    wide[:, 2:2 + proj.shape[1]] = proj
    wide = dev(wide)
    rotd = {"base": 777.0, "dims": rot}
    if scaling:
        rotd["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    freq, mag = (plain.rotary_frequencies(rotd) if rot else (None, 1.0))
    cache = PagedKV(3, 4096, G, dk, dv, dtype)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    qo = torch.full((T, H * dk), float("nan"), dtype=dtype, device=DEV)
    kw = dict(norm=norm, q_norm=dev(wq) if norm else None, k_norm=dev(wk) if norm else None, eps=eps,
              interleaved=pairing == "interleaved", magnitude=mag)
    fr = dev(torch.tensor(freq, dtype=torch.float64)) if rot else None
    ops.qkv_rope_append(wide[:, 2:2 + proj.shape[1]], 0, H * dk, H * dk + (G * dk if own_values else 0), fr, rot, qo, cache.k, cache.v, cache.table,
                        dev(torch.tensor(slot_of), torch.int32), dev(torch.tensor(positions), torch.int32), T, H, G, dk, dv, True, err, **kw)
    assert int(err.item()) == 0
    pos = torch.tensor(positions)

    def want(x, heads, w):
        x = x.double().view(T, heads, dk)
        if norm == "head":
            x = plain.rms_norm(x, w.double(), eps)
        elif norm == "all":
            x = plain.rms_norm(x.reshape(T, -1), w.double(), eps).view(T, heads, dk)
        return plain.rotate(x, pos, rotd, pairing) if rot else x
    close(qo.view(T, H, dk), want(q, H, wq), tol, "queries")
    want_k, want_v = want(k, G, wk), (v if own_values else k).double().view(T, G, dv)
    for t, (s, p) in enumerate(zip(slot_of, positions)):
        blk = int(cache.table[s, p // 64])
        close(cache.k[blk, :, p % 64], want_k[t], tol, f"key of token {t}")
        close(cache.v[blk, :, p % 64], want_v[t], tol, f"value of token {t}")
    written = (~torch.isnan(cache.k.float())).sum().item()
    assert written == T * G * dk
    # a layer that reads another layer's cache: the queries only
    only_q = torch.full((T, H * dk + 3), float("nan"))
    only_q[:, 1:1 + H * dk] = q
    only_q = dev(only_q)
    before = cache.k.clone()
    qo2 = torch.full_like(qo, float("nan"))
    kw["k_norm"] = None
    ops.qkv_rope_append(only_q[:, 1:1 + H * dk], 0, 0, 0, fr, rot, qo2, cache.k, cache.v, cache.table, dev(torch.tensor(slot_of), torch.int32),
                        dev(torch.tensor(positions), torch.int32), T, H, G, dk, dv, False, err, **kw)
    assert torch.equal(qo2.float().cpu(), qo.float().cpu()) and torch.equal(torch.nan_to_num(before.float()), torch.nan_to_num(cache.k.float()))


def attention_case(H, G, dk, window, keep, softcap, sinks, dtype, lens, seed):
    """Random queries, keys and values (bfloat16 values, exact in both dtypes) for sequences of `lens` tokens.  For the LAST
    query of every sequence four keys are made loud through the first query head of each key/value head: the oldest key
    inside the window and the last kept key (both visible) and, louder still, the key just outside the window and the
    first key that is not kept (both invisible, where they exist and lie apart)."""
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    rd = lambda *shape: torch.randn(*shape, generator=g).bfloat16().double()   # noqa: E731
    q, k, v = rd(T, H, dk), rd(T, G, dk), rd(T, G, dk)
    start = 0
    for n in lens:
        last = start + n - 1
        inside = max(0, n - window) if window else 0
        for hk in range(G):
            h = hk * (H // G)
            unit = q[last, h] / float(q[last, h].norm())
            k[start + inside, hk] = (5.0 * unit).bfloat16().double()
            if inside > keep:
                k[start + inside - 1, hk] = (8.0 * unit).bfloat16().double()          # just outside the window, and not kept
                if keep > 0:
                    k[start + keep - 1, hk] = (5.5 * unit).bfloat16().double()        # the last kept key
                    if inside - 1 > keep:
                        k[start + keep, hk] = (8.5 * unit).bfloat16().double()        # the first that is not kept
        start += n
    sink = (torch.randn(H, generator=g) * 2.0 + 3.0).double() if sinks else None
    mask = {"size": window, "keep_first": keep} if window else None
    want, start = [], 0
    for n in lens:
        sl = slice(start, start + n)
        want.append(plain.attend(q[sl], k[sl], v[sl], 0.5, mask, softcap, sink))
        start += n
    return q, k, v, sink, torch.cat(want)


def run_attention(q, k, v, sink, lens, window, keep, softcap, dtype, tail, splits=None, gate=None):
    """Everything is appended to a NaN-filled cache under a permuted block table; then the last `tail` tokens of every
    sequence (None: all of them, by the kernel that takes a warp per token and head) attend.  gate: float32 [T, H] logits of
    a gate per head, handed over as a range of columns of wider rows."""
    from vlrf_b200.csrc import ops
    from vlrf_b200.parts.context import Workspace
    T, H, dk = q.shape
    G = k.shape[1]
    slot_of = [s for s, n in enumerate(lens) for _ in range(n)]
    positions = [p for n in lens for p in range(n)]
    cache = PagedKV(len(lens), max(lens), G, dk, dk, dtype)
    proj = dev(torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1))
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    qo = torch.full((T, H * dk), float("nan"), dtype=dtype, device=DEV)
    tok_slot, tok_pos = dev(torch.tensor(slot_of), torch.int32), dev(torch.tensor(positions), torch.int32)
    ops.qkv_rope_append(proj, 0, H * dk, H * dk + G * dk, None, 0, qo, cache.k, cache.v, cache.table, tok_slot, tok_pos, T, H, G, dk, dk, True, err)
    sk = dev(sink) if sink is not None else None
    extra = dict(softcap=softcap or 0.0, keep_first=keep, sink=sk)

    def gate_rows(rows):
        if gate is None:
            return None
        wide = torch.full((len(rows), H + 5), float("nan"))
        wide[:, 2:2 + H] = gate[torch.tensor(rows)].float()
        return dev(wide)[:, 2:2 + H]
    if tail is None:
        out = torch.full((T, H * dk), float("nan"), dtype=dtype, device=DEV)
        ops.attention_window(qo, cache.k, cache.v, cache.table, tok_slot, tok_pos, out, T, H, G, dk, dk, 0.5, window, 1.0, err,
                             gate=gate_rows(list(range(T))), **extra)
        rows = list(range(T))
    else:
        rows, seq_start, seq_pos0, start = [], [0], [], 0
        for n in lens:
            m = min(tail, n)
            rows += list(range(start + n - m, start + n))
            seq_start.append(seq_start[-1] + m)
            seq_pos0.append(n - m)
            start += n
        idx = torch.tensor(rows)
        ctx = types.SimpleNamespace(
            n_tokens=len(rows), n_seqs=len(lens), max_new=min(tail, max(lens)), max_context=max(lens), ws=Workspace(DEV), dev_err=err,
            tok_slot=dev(torch.tensor(slot_of)[idx], torch.int32), tok_pos=dev(torch.tensor(positions)[idx], torch.int32),
            seq_slot=dev(torch.arange(len(lens)), torch.int32), seq_start=dev(torch.tensor(seq_start), torch.int32),
            seq_pos0=dev(torch.tensor(seq_pos0), torch.int32))
        out = torch.full((len(rows), H * dk), float("nan"), dtype=dtype, device=DEV)
        if splits:
            os.environ["VLRF_B200_DECODE_SPLITS"] = str(splits)
        try:
            ops.attention_window_step(qo[idx.to(DEV)].contiguous(), cache.k, cache.v, cache.table, out, ctx, H, G, dk, dk, 0.5, window, 1.0,
                                      gate=gate_rows(rows), **extra)
        finally:
            os.environ.pop("VLRF_B200_DECODE_SPLITS", None)
    assert int(err.item()) == 0
    return out.view(len(rows), H, dk), rows


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H,G,dk,window,keep,softcap,sinks", [
    (4, 1, 16, 40, 5, 6.0, True), (6, 2, 32, 70, 0, 10.0, True), (4, 4, 8, 64, 64, None, True), (8, 2, 8, 33, 70, 30.0, True),
    (5, 1, 12, 7, 3, 4.0, True), (3, 3, 64, 130, 1, None, False), (2, 1, 24, 0, 0, 9.0, True), (16, 1, 64, 100, 24, 18.0, False),
    (2, 2, 128, 65, 63, 12.0, True)])
def test_attention_at_the_edges(H, G, dk, window, keep, softcap, sinks, dtype, tol):
    """Sequences of 1, 2, 64, 65, 129, 200 and 333 tokens in one step: as one prompt step (both kernels), as a later portion
    of 70 and of 3 tokens, and as a decode step whose contexts are whole, cut in 2 and cut in 5 parts.  Where the shape has
    sinks it also has a gate per head, applied by the attention kernels themselves."""
    lens = [1, 2, 64, 65, 129, 200, 333]
    q, k, v, sink, want = attention_case(H, G, dk, window, keep, softcap, sinks, dtype, lens, dk * 7 + window)
    gate = None
    if sinks:
        gate = torch.randn(sum(lens), H, generator=torch.Generator().manual_seed(dk)).double() * 2.0
        want = want * torch.sigmoid(gate.float().double())[:, :, None]
    got, rows = run_attention(q, k, v, sink, lens, window, keep, softcap, dtype, None, gate=gate)
    close(got, want, tol, "a warp per token and head")
    for tail, splits in ((10 ** 6, None), (70, None), (3, None), (1, 1), (1, 2), (1, 5)):
        got, rows = run_attention(q, k, v, sink, lens, window, keep, softcap, dtype, tail, splits, gate=gate)
        close(got, want[torch.tensor(rows)], tol, f"the last {tail} tokens, contexts in {splits} parts")


def test_a_sink_takes_its_share_and_an_edge_key_would_show():
    """The plain implementation's own edges, on the inputs above: dropping the sinks, moving the window by one or keeping
    one token more or fewer changes the expected result by far more than the kernels' tolerance."""
    lens = [200, 333]
    q, k, v, sink, want = attention_case(4, 1, 16, 40, 5, 6.0, True, torch.float32, lens, 1)
    last = [199, 532]

    def again(mask, sk):
        out, start = [], 0
        for n in lens:
            out.append(plain.attend(q[start:start + n], k[start:start + n], v[start:start + n], 0.5, mask, 6.0, sk))
            start += n
        return torch.cat(out)[last]
    for mask, sk in (({"size": 41, "keep_first": 5}, sink), ({"size": 39, "keep_first": 5}, sink), ({"size": 40, "keep_first": 6}, sink),
                     ({"size": 40, "keep_first": 4}, sink), ({"size": 40, "keep_first": 5}, None)):
        assert float((again(mask, sk) - want[last]).abs().max() / want.abs().max()) > 0.05, (mask, sk is None)


def bigram_step(table, pairs, cfgb, scale, kept, entries, V):
    """One step of the bigram embedding: entries [(slot, position of the first token, tokens)]; slot −1: a padding row."""
    from vlrf_b200.csrc import ops
    tokens, slots, poss, seq_start = [], [], [], [0]
    for slot, p0, toks in entries:
        tokens += toks
        slots += [slot] * len(toks)
        poss += list(range(p0, p0 + len(toks))) if slot >= 0 else [0] * len(toks)
        seq_start.append(len(tokens))
    T = len(tokens)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ctx = types.SimpleNamespace(n_tokens=T, n_seqs=len(entries), tokens=dev(torch.tensor(tokens), torch.int32),
                                tok_slot=dev(torch.tensor(slots), torch.int32), tok_pos=dev(torch.tensor(poss), torch.int32),
                                seq_start=dev(torch.tensor(seq_start), torch.int32), dev_err=err)
    out = torch.full((T + 1, table.shape[1]), float("nan"), device=DEV)
    ops.embed_bigram(table, pairs, cfgb["buckets"], cfgb["mul_prev"], cfgb["mul_cur"], scale, kept, ctx, out)
    assert int(err.item()) == 0 and torch.isnan(out[T]).all()
    return out[:T].cpu()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V,d,buckets,mul_prev,mul_cur", [(301, 96, 53, 31, 5), (64, 40, 1, 0, 3), (50000, 33, 4099, 50021, 7919)])
def test_bigram_embedding_over_steps(V, d, buckets, mul_prev, mul_cur, dtype):
    """Three sequences in slots 3, 0 and 5 of a table whose other slots hold impossible tokens: prompts of 5, 8 and 1
    tokens, then portions of even and odd lengths and single tokens in changing order with a padding row between them, and
    a step of single tokens run twice.  Every row against the hash written out over the whole sequences."""
    g = torch.Generator().manual_seed(V)
    table, pairs = torch.randn(V, d, generator=g).to(dtype), torch.randn(buckets + 1, d, generator=g).to(dtype)
    cfgb = {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}
    seqs = {3: torch.randint(0, V, (40,), generator=g).tolist(), 0: torch.randint(0, V, (40,), generator=g).tolist(),
            5: torch.randint(0, V, (40,), generator=g).tolist()}
    want = {s: (table.double()[ids] * 1.5 + pairs.double()[plain.bigram_rows(ids, buckets, mul_prev, mul_cur)]) for s, ids in seqs.items()}
    kept = torch.full((7, 2), 1 << 30, dtype=torch.int32, device=DEV)
    for s in seqs:
        kept[s] = 0
    at = {s: 0 for s in seqs}
    td, pd = dev(table, dtype), dev(pairs, dtype)
    plan = [[(3, 5), (0, 8), (5, 1)], [(0, 2), (-1, 1), (3, 1), (5, 4)], [(5, 1), (3, 3)], [(3, 1), (-1, 1), (0, 1), (5, 1)],
            [(0, 7), (5, 2)], [(5, 1), (0, 1), (3, 1)], [(3, 6), (0, 1)], [(0, 1), (3, 1), (5, 1)]]
    for step, parts in enumerate(plan):
        entries = [(s, at[s] if s >= 0 else 0, seqs[s][at[s]:at[s] + n] if s >= 0 else [0] * n) for s, n in parts]
        runs = 2 if all(n == 1 for _, n in parts) else 1             # a step of single tokens may run twice
        for _ in range(runs):
            got = bigram_step(td, pd, cfgb, 1.5, kept, entries, V)
            r = 0
            for s, n in parts:
                if s >= 0:
                    close(got[r:r + n], want[s][at[s]:at[s] + n], 1e-6, f"step {step}, slot {s}")
                r += n
        for s, n in parts:
            if s >= 0:
                at[s] += n
    assert all(int(kept[s, 0]) == 1 << 30 for s in (1, 2, 4, 6))


@pytest.mark.parametrize("E,top", [(5, 2), (11, 4), (3, 3), (7, 1), (40, 6), (130, 8)])
def test_router_by_sigmoid_scores(E, top):
    from vlrf_b200.csrc import ops
    g = torch.Generator().manual_seed(E)
    T = 37
    z = torch.randn(T, E + 3, generator=g) * 2.0
    corr = torch.randn(E, generator=g) * 0.7
    z[5, :E] = 0.3                                     # all scores equal: the correction alone decides, ties to the lower index
    z[6, :E] = torch.linspace(-1, 1, E)
    slot = torch.zeros(T, dtype=torch.int32)
    slot[9] = -1
    ids, rank = (torch.full((T, top), -7, dtype=torch.int32, device=DEV) for _ in range(2))
    wts = torch.full((T, top), float("nan"), device=DEV)
    counts = torch.zeros(E, dtype=torch.int32, device=DEV)
    ops.moe_route_scored(dev(z), E, top, 1, 1, 0, 1.0, dev(corr), dev(slot), ids, wts, rank, counts, T, scoring="sigmoid")
    w = {"r.router": torch.eye(E, dtype=torch.float64), "r.correction": corr.double()}
    want_idx, want_w = plain.route(z[:, :E].double(), w, "r.", {"router": {"top": top}})
    live = [t for t in range(T) if t != 9]
    assert torch.equal(ids.cpu()[live].long(), want_idx[live])
    close(wts[live], want_w[live], 1e-6, "weights")
    assert ids[9].tolist() == [-1] * top and float(wts[9].abs().sum()) == 0.0
    assert torch.equal(counts.cpu().long(), torch.bincount(want_idx[live].flatten(), minlength=E))
    # the weights are the scores themselves: not renormalized, and blind to the correction
    assert float((want_w.sum(1) - 1.0).abs().min()) > 1e-3 or top == 1


@pytest.mark.parametrize("a_dt,o_dt", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("cols,lead", [(40, 0), (96, 0), (36, 3)])
def test_gates(a_dt, o_dt, cols, lead):
    from vlrf_b200.csrc import ops
    g = torch.Generator().manual_seed(cols)
    rows = 19
    a, b = (torch.randn(rows, cols, generator=g) * 3.0).to(a_dt), (torch.randn(rows, cols, generator=g) * 3.0).to(a_dt)
    wide = torch.full((rows + 1, 2 * cols + lead + 1), float("nan"), dtype=a_dt)
    wide[:rows, lead:lead + cols], wide[:rows, lead + cols:lead + 2 * cols] = a, b
    wide = wide.to(DEV)
    tol = 1e-6 if o_dt == torch.float32 else 5e-3
    out = torch.full((rows + 1, cols), float("nan"), dtype=o_dt, device=DEV)
    ops.gate_mul_clamped(wide[:, lead:lead + cols], wide[:, lead + cols:lead + 2 * cols], out, 1.25, 1.702, rows, cols)
    gd, ud = a.double().clamp(max=1.25), b.double().clamp(-1.25, 1.25)
    close(out[:rows], gd * torch.sigmoid(1.702 * gd) * (ud + 1.0), tol, "bounded gate")
    assert torch.isnan(out[rows].float()).all()
    if a_dt == torch.float32:
        out.fill_(float("nan"))
        ops.gate_mul(wide[:, lead:lead + cols], wide[:, lead + cols:lead + 2 * cols], out, "gelu_tanh", rows, cols)
        close(out[:rows], plain.gelu_tanh(a.double()) * b.double(), tol, "GELU gate")
    lg = torch.randn(4, 31, generator=g)
    ld = dev(lg)
    ops.scale_values(ld, 3, 0.7)
    close(ld[:3], lg[:3].double() * 0.7, 1e-6, "scaled")
    assert torch.equal(ld[3].cpu(), lg[3])
    # in place, as the experts' feed-forward calls it on wider rows
    if a_dt == o_dt:
        ops.gate_mul_clamped(wide[:, lead:lead + cols], wide[:, lead + cols:lead + 2 * cols], wide[:, lead:lead + cols], 0.5, 1.0, rows, cols)
        gd, ud = a.double().clamp(max=0.5), b.double().clamp(-0.5, 0.5)
        close(wide[:rows, lead:lead + cols], gd * torch.sigmoid(gd) * (ud + 1.0), tol, "bounded gate in place")
