"""Each mechanism of the Rakelorn design alone: the kernel against the plain function on inputs of its own — the norm with
its token shift and the gated recurrence over steps of every cut (both copies of their states, other slots full of NaN,
padding rows), the router by scores with groups, a correction and identity experts, the weighted sum with experts that
return their input, the gate per head, the rotation of neighbouring pairs, the vector added to every row."""
import math
import types

import pytest
import torch

import plain_rakelorn as plain

pytestmark = pytest.mark.gpu

DT = [torch.float32, torch.bfloat16]


def tol(dt):
    return 2e-5 if dt == torch.float32 else 1.2e-2


def close(got, want, t, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    assert math.isfinite(err) and err <= t, f"{what}: error {err:.3e} above {t:.1e}"


def dev(t, dt=None):
    return t.to("cuda", dt if dt is not None else t.dtype).contiguous()


def step_ctx(runs, pad_rows=()):
    """A step's tables: `runs` = [(slot, first position, tokens)], in row order; `pad_rows`: indices (among the sequences)
    at which a padding row of one token (slot −1) is put in."""
    slot, pos, seq_slot, seq_start, seq_pos0 = [], [], [], [0], []
    runs = list(runs)
    for i in sorted(pad_rows, reverse=True):
        runs.insert(i, (-1, 0, 1))
    for s, p0, n in runs:
        slot += [s] * n
        pos += list(range(p0, p0 + n))
        seq_slot.append(s)
        seq_pos0.append(p0)
        seq_start.append(seq_start[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    return types.SimpleNamespace(n_tokens=len(slot), tok_slot=i32(slot), tok_pos=i32(pos), n_seqs=len(runs), seq_slot=i32(seq_slot),
                                 seq_start=i32(seq_start), seq_pos0=i32(seq_pos0), max_new=max(n for _, _, n in runs)), runs


#: three sequences in slots 4, 1 and 6 of 8, cut into steps so that every state copy is read and written: a prompt step of
#: unequal runs, single tokens (twice, so that a step begins at an odd and at an even position), portions of 2, 3 and 6
STEPS = [[5, 8, 1], [1, 1, 1], [1, 1, 1], [2, 3, 6], [1, 1, 1], [4, 2, 7]]
SLOTS = [4, 1, 6]


def run_steps(fn, lengths_done, n_slots, width, out_dtype):
    """Drive `fn(ctx, rows_of_each_sequence) -> out rows` over STEPS; returns each sequence's output rows in order."""
    outs = [[] for _ in SLOTS]
    for k, step in enumerate(STEPS):
        ctx, runs = step_ctx([(SLOTS[i], lengths_done[i], n) for i, n in enumerate(step)], pad_rows=(1,) if k % 2 else ())
        out = fn(ctx, runs)
        at = 0
        for s, p0, n in runs:
            if s >= 0:
                outs[SLOTS.index(s)].append(out[at:at + n].float().cpu())
            at += n
        for i, n in enumerate(step):
            lengths_done[i] += n
    return [torch.cat(o) for o in outs]


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("d", [96, 100, 1024, 2048, 4100, 8200])      # (rows held by 1, 2 and 4 quads a thread, by more threads; too wide: a warp a token)
def test_norm_with_token_shift_over_steps(d, dt):
    from vlrf_b200.csrc import ops
    g = torch.Generator().manual_seed(d)
    total = [sum(s[i] for s in STEPS) for i in range(3)]
    xs = [torch.randn(n, d, generator=g, dtype=torch.float64) * torch.linspace(0.1, 5, d, dtype=torch.float64) for n in total]
    w = torch.full((d,), 1.3, dtype=torch.float64)
    mu = torch.rand(d, generator=g, dtype=torch.float64)
    mu[0], mu[1] = 0.0, 1.0
    want = [plain.token_shift(plain.scalar_rms_norm(x, 1.3, 1e-5), mu) for x in xs]
    state = torch.full((8, 2, d), float("nan"), device="cuda")
    for s in SLOTS:
        state[s] = 0.0                                    # (a slot is zeroed when a sequence takes it)
    wd, mud = dev(w, torch.float32), dev(mu, torch.float32)
    done = [0, 0, 0]

    def fn(ctx, runs):
        x = torch.cat([xs[SLOTS.index(s)][p0:p0 + n] if s >= 0 else torch.full((n, d), float("nan"), dtype=torch.float64) for s, p0, n in runs])
        out = torch.full((ctx.n_tokens, d), 7.0, dtype=dt, device="cuda")
        ops.rmsnorm_shift(dev(x, torch.float32), wd, mud, 1e-5, state, ctx, out)
        return out

    got = run_steps(fn, done, 8, d, dt)
    for i in range(3):
        close(got[i], want[i], tol(dt), f"sequence {i}")
    # the kept rows: the unshifted normed row of each sequence's last token, in the copy of the parity of its length
    for i, s in enumerate(SLOTS):
        close(state[s, total[i] & 1], plain.scalar_rms_norm(xs[i][-1:], 1.3, 1e-5)[0], 2e-6, "kept row")
    others = [s for s in range(8) if s not in SLOTS]
    assert torch.isnan(state[others]).all(), "a state of another slot was written"


def test_a_decode_step_of_the_shifted_norm_may_run_twice():
    from vlrf_b200.csrc import ops
    d = 64
    g = torch.Generator().manual_seed(1)
    x = dev(torch.randn(2, d, generator=g), torch.float32)
    w, mu = torch.ones(d, device="cuda"), torch.full((d,), 0.5, device="cuda")
    state = dev(torch.randn(3, 2, d, generator=g), torch.float32)
    ctx, _ = step_ctx([(2, 7, 1), (0, 4, 1)])
    a, b = torch.zeros(2, d, device="cuda"), torch.zeros(2, d, device="cuda")
    ops.rmsnorm_shift(x, w, mu, 1e-5, state, ctx, a)
    ops.rmsnorm_shift(x, w, mu, 1e-5, state, ctx, b)
    assert torch.equal(a, b)


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("W", [52, 112, 1024])
def test_gated_recurrence_over_steps(W, dt):
    from vlrf_b200.csrc import ops
    g = torch.Generator().manual_seed(W)
    total = [sum(s[i] for s in STEPS) for i in range(3)]
    ld = 3 * W + 5                                        # (the three ranges inside wider rows, not side by side)
    offs = (2, 2 * W + 5, W + 3)
    projs = [torch.randn(n, ld, generator=g, dtype=torch.float64) * 2 for n in total]
    want = []
    for p in projs:
        a, u, gg = (p[:, o:o + W] for o in offs)
        cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
        S = plain.mingru_scan(torch.sigmoid(a), cand)
        want.append(S * gg * torch.sigmoid(gg))
    state = torch.full((8, 2, W), float("nan"), device="cuda")
    for s in SLOTS:
        state[s] = 0.0
    done = [0, 0, 0]

    def fn(ctx, runs):
        p = torch.cat([projs[SLOTS.index(s)][p0:p0 + n] if s >= 0 else torch.full((n, ld), float("nan"), dtype=torch.float64) for s, p0, n in runs])
        out = torch.zeros(ctx.n_tokens, W, dtype=dt, device="cuda")
        ops.mingru_scan(dev(p, torch.float32), offs[0], offs[1], offs[2], W, state, ctx, out)
        return out

    got = run_steps(fn, done, 8, W, dt)
    for i in range(3):
        close(got[i], want[i], tol(dt), f"sequence {i}")
    others = [s for s in range(8) if s not in SLOTS]
    assert torch.isnan(state[others]).all(), "a state of another slot was written"


@pytest.mark.parametrize("dt", DT)
def test_gated_recurrence_of_long_unequal_prompts_in_one_step(dt):
    """Prompts long enough that several CTAs share a sequence's tokens (the longest decides how many), beside a short one
    and a single token; then a second portion that begins at an odd position, from the states the first left."""
    from vlrf_b200.csrc import ops
    W = 70
    first, second = [1301, 37, 1, 600], [260, 3, 1030, 1]
    g = torch.Generator().manual_seed(11)
    projs = [torch.randn(a + b, 3 * W, generator=g, dtype=torch.float64) * 2 for a, b in zip(first, second)]
    for p in projs:
        p[:, :W] -= 2.0                                    # (gates that keep: a wrong state at a run's start shows for long)
    want = []
    for p in projs:
        a, u, gg = p[:, :W], p[:, W:2 * W], p[:, 2 * W:]
        S = plain.mingru_scan(torch.sigmoid(a), torch.where(u >= 0, u + 0.5, torch.sigmoid(u)))
        want.append(S * gg * torch.sigmoid(gg))
    slots = [5, 0, 3, 2]
    state = torch.full((6, 2, W), float("nan"), device="cuda")
    for s in slots:
        state[s] = 0.0
    got = [[] for _ in slots]
    for part, lens in enumerate((first, second)):
        p0s = [0] * 4 if part == 0 else first
        ctx, _ = step_ctx([(s, p0, n) for s, p0, n in zip(slots, p0s, lens)])
        rows = torch.cat([p[p0:p0 + n] for p, p0, n in zip(projs, p0s, lens)])
        out = torch.zeros(ctx.n_tokens, W, dtype=dt, device="cuda")
        ops.mingru_scan(dev(rows, torch.float32), 0, W, 2 * W, W, state, ctx, out)
        at = 0
        for i, n in enumerate(lens):
            got[i].append(out[at:at + n].float().cpu())
            at += n
    for i in range(4):
        close(torch.cat(got[i]), want[i], tol(dt), f"sequence {i}")
    assert torch.isnan(state[[1, 4]]).all(), "a state of another slot was written"


def test_gated_recurrence_keeps_a_far_token():
    """A channel whose gate is nearly shut after the first token carries that token's candidate over 700 tokens of a prompt
    step (many runs of warps) and over the decode steps behind it; an open channel beside it forgets at once."""
    from vlrf_b200.csrc import ops
    W, n = 40, 700
    g = torch.Generator().manual_seed(3)
    p = torch.randn(n + 3, 3 * W, generator=g, dtype=torch.float64)
    p[1:, 0] = -30.0                                       # channel 0: z ≈ 1e-13 behind the first token
    p[0, 0], p[0, W] = 30.0, 41.5                          # the first token writes 42 there
    p[:, 1] = 30.0                                         # channel 1: z ≈ 1, the state is the newest candidate
    a, u, gg = p[:, :W], p[:, W:2 * W], p[:, 2 * W:]
    S = plain.mingru_scan(torch.sigmoid(a), torch.where(u >= 0, u + 0.5, torch.sigmoid(u)))
    want = S * gg * torch.sigmoid(gg)
    assert abs(float(S[-1, 0]) - 42.0) < 1e-6
    state = torch.zeros(2, 2, W, device="cuda")
    pd = dev(p, torch.float32)
    out = torch.zeros(n + 3, W, device="cuda")
    ctx, _ = step_ctx([(1, 0, n)])
    ops.mingru_scan(pd[:n], 0, W, 2 * W, W, state, ctx, out[:n])
    for k in range(3):
        ctx, _ = step_ctx([(1, n + k, 1)])
        ops.mingru_scan(pd[n + k:n + k + 1], 0, W, 2 * W, W, state, ctx, out[n + k:n + k + 1])
    close(out, want, 2e-5, "outputs")
    close(state[1, (n + 3) & 1], S[-1], 2e-6, "the kept state")


@pytest.mark.parametrize("E,n_id,top,count,keep", [(6, 2, 3, 4, 2), (5, 1, 2, 3, 1), (4, 0, 1, 1, 1), (0, 3, 2, 1, 1), (3, 3, 2, 3, 2),
                                                   (60, 4, 6, 8, 3), (7, 2, 2, 3, 3), (100, 4, 5, 8, 4), (250, 6, 8, 16, 5)])      # (1, 2, 4 and 16 logits a lane)
def test_router_by_scores(E, n_id, top, count, keep):
    from vlrf_b200.csrc import ops
    n_out = E + n_id
    g = torch.Generator().manual_seed(n_out * 7 + top)
    T = 41
    z = torch.randn(T, n_out + 2, generator=g, dtype=torch.float64) * 2
    z[4, :n_out] = 1.5                                     # all equal: the lowest groups and indices win
    corr = 0.1 * torch.randn(n_out, generator=g, dtype=torch.float64)
    corr_t = [corr] * T
    slot = torch.zeros(T, dtype=torch.int32)
    slot[10] = -1                                          # a padding row chooses nothing
    r = {"top": top, "scale": 1.7, "groups": {"count": count, "keep": keep}}
    zf = z.float().double()                                # (what the kernel is given)
    want_ids, want_w = plain.route(zf[:, :n_out], corr.float().double(), r)
    ids = torch.zeros(T, top, dtype=torch.int32, device="cuda"); rank = torch.zeros_like(ids)
    wts = torch.zeros(T, top, device="cuda")
    counts = torch.zeros(max(E, 1), dtype=torch.int32, device="cuda")
    ops.moe_route_scored(dev(z, torch.float32), n_out, top, count, keep, n_id, 1.7, dev(corr, torch.float32), slot.cuda(), ids, wts, rank, counts, T)
    got = ids.cpu()
    live = [t for t in range(T) if t != 10]
    for t in live:
        assert got[t].tolist() == [e if e < E else -2 for e in want_ids[t]], (t, got[t].tolist(), want_ids[t])
        close(wts[t], torch.tensor(want_w[t]), 2e-6, "weights")
    assert got[10].tolist() == [-1] * top
    n_of = torch.bincount(torch.tensor([e for t in live for e in want_ids[t] if e < E], dtype=torch.long), minlength=max(E, 1))
    assert counts.cpu().tolist() == n_of.tolist()
    # the ranks of an expert's pairs are 0 … count − 1, each once
    rk = rank.cpu()
    for e in range(E):
        mine = sorted(int(rk[t, j]) for t in live for j in range(top) if got[t, j] == e)
        assert mine == list(range(int(n_of[e])))


def test_router_with_negative_choice_scores_and_a_nan():
    """A correction so negative that every choice score is below zero: a dropped group's experts must still lose (they count
    as −infinity, not as 0); a NaN logit is never chosen before a number."""
    from vlrf_b200.csrc import ops
    n_out, top = 6, 2
    z = torch.log(torch.tensor([[0.05, 0.30, 0.25, 0.20, 0.15, 0.05], [0.2, 0.2, 0.1, 0.1, 0.3, 0.1]], dtype=torch.float64))
    z[1, 4] = float("nan")
    corr = torch.full((n_out,), -5.0, dtype=torch.float64)
    ids = torch.zeros(2, top, dtype=torch.int32, device="cuda"); rank = torch.zeros_like(ids)
    wts = torch.zeros(2, top, device="cuda"); counts = torch.zeros(n_out, dtype=torch.int32, device="cuda")
    ops.moe_route_scored(dev(z, torch.float32), n_out, top, 3, 1, 0, 1.0, dev(corr, torch.float32), None, ids, wts, rank, counts, 2)
    assert ids.cpu()[0].tolist() == [1, 0] and ids.cpu()[1].tolist() == [0, 1]
    close(wts[0], torch.tensor([0.30, 0.05]), 1e-6, "weights")


def test_weighted_sum_with_experts_that_return_their_input():
    from vlrf_b200.csrc import ops
    g = torch.Generator().manual_seed(5)
    T, top, width = 9, 3, 20
    for hd in DT:
        ids = torch.tensor([[0, -2, 1], [-2, -2, 2], [-1, -1, -1]] * 3, dtype=torch.int32, device="cuda")
        row_of = torch.tensor([[0, -1, 1], [-1, -1, 2], [-1, -1, -1]] * 3, dtype=torch.int32, device="cuda")
        wts = dev(torch.rand(T, top, generator=g), torch.float32)
        eo = dev(torch.randn(3, width, generator=g), torch.float32)
        h = dev(torch.randn(T, width, generator=g), hd)
        y = torch.ones(T, width, device="cuda")
        ops.moe_combine(eo, row_of, wts, top, None, None, y, T, residual=y, ids=ids, h=h)
        want = torch.ones(T, width, dtype=torch.float64)
        for t in range(T):
            for j in range(top):
                if int(row_of[t, j]) >= 0:
                    want[t] += float(wts[t, j]) * eo[int(row_of[t, j])].double().cpu()
                elif int(ids[t, j]) == -2:
                    want[t] += float(wts[t, j]) * h[t].double().cpu()
        close(y, want, 1e-6, "combine")


@pytest.mark.parametrize("H,vdim", [(3, 24), (5, 7), (16, 64)])
def test_gate_per_head(H, vdim):
    from vlrf_b200.csrc import ops
    g = torch.Generator().manual_seed(H)
    T = 11
    wide = torch.randn(T, H + 9, generator=g, dtype=torch.float64)
    b = torch.randn(T, H * vdim, generator=g, dtype=torch.float64)
    want = torch.sigmoid(wide[:, 4:4 + H]).repeat_interleave(vdim, dim=1) * b
    a32 = dev(wide, torch.float32)
    for dt in DT:
        bd = dev(b, dt)
        ops.gate_mul(a32[:, 4:4 + H], bd, bd, "sigmoid", T, H * vdim, per=vdim)          # in place, the gate a range of wider rows
        close(bd, want, tol(dt), "gate per head")


@pytest.mark.parametrize("R,dims", [(16, 16), (16, 8), (6, 6), (32, 2)])
def test_rotation_of_neighbouring_pairs_in_cache_rows_and_queries(R, dims):
    from vlrf_b200.cache.sequence_cache import BLOCK_TOKENS as BT
    from vlrf_b200.csrc import ops
    from vlrf_b200.parts import RotaryPositions
    g = torch.Generator().manual_seed(R + dims)
    C, H, dim = 24, 3, 10
    rot = RotaryPositions(777.0, dims, "cuda", pairing="interleaved")
    positions = torch.tensor([0, 1, 63, 64, 130], dtype=torch.int32)
    T = len(positions)
    proj = torch.randn(T, C + R + 3, generator=g, dtype=torch.float64)
    w = 1 + 0.2 * torch.randn(C, generator=g, dtype=torch.float64)
    cache = torch.full((4, BT, C + R), float("nan"), device="cuda")
    table = torch.tensor([[3, 0, 2, 1]], dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.latent_append(dev(proj, torch.float32), C, R, dev(w, torch.float32), 1e-5, rot.inv_freq, dims, cache, table,
                      torch.zeros(T, dtype=torch.int32, device="cuda"), positions.cuda(), T, err, interleaved=True)
    want_c = plain.rms_norm(proj[:, :C], w, 1e-5)
    want_r = plain.rotate_pairs(proj[:, C:C + R], positions, 777.0, dims)
    for t, p in enumerate(positions.tolist()):
        row = cache[int(table[0, p // BT]), p % BT]
        close(row[:C], want_c[t], 2e-6, "latent")
        close(row[C:], want_r[t], 2e-5, "rotated key part")
    assert int(err.item()) == 0 and int(torch.isfinite(cache).all(dim=2).sum()) == T
    q = torch.randn(T, H * (dim + R), generator=g, dtype=torch.float64)
    qn = torch.zeros(T, H * dim, device="cuda"); qp = torch.zeros(T, H * (C + R), device="cuda")
    ops.latent_q_rows(dev(q, torch.float32), H, dim, R, rot.inv_freq, dims, positions.cuda(), qn, qp, C, T, interleaved=True)
    q3 = q.reshape(T, H, dim + R)
    close(qn, q3[..., :dim].reshape(T, -1), 1e-6, "unrotated parts")
    close(qp.view(T, H, C + R)[..., C:], plain.rotate_pairs(q3[..., dim:], positions, 777.0, dims), 2e-5, "rotated parts")


def test_vector_added_to_every_row():
    from vlrf_b200.csrc import ops
    x = torch.arange(5 * 12, dtype=torch.float32, device="cuda").reshape(5, 12).clone()
    keep = x.clone()
    v = torch.arange(10, dtype=torch.float32, device="cuda") * 0.5
    ops.add_row_vector(x[:, :10], v, 4)
    assert torch.equal(x[:4, :10], keep[:4, :10] + v) and torch.equal(x[4], keep[4]) and torch.equal(x[:, 10:], keep[:, 10:])
