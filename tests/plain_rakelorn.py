"""A plain, slow implementation of the Rakelorn design in float64, one function per mechanism, written from the
design's equations and sharing no code with the package (it reads model folders with the tests' own reader).

Notation: T tokens, width d.  Linear weights are [out, in] and applied as x · Wᵀ.  Everything runs over a whole
sequence from its first token, so there is no cache and no state here: the recurrence and the token shift simply
start from zeros.
"""
from __future__ import annotations

import math

import torch

from plain_gpt2 import read_model_dir  # noqa: F401  (the tests' own reader of config.json + model.safetensors)


def scalar_rms_norm(x, g, eps):
    """x / sqrt(mean(x²) + eps) · g with one number g for the whole row."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * g


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def token_shift(h, mu):
    """h_t ← h_t + (h_(t−1) − h_t) · mu, with the unshifted h of the token before and zeros before the first."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (prev - h) * mu


def rotate_pairs(v, positions, base, dims):
    """v [T, …, n]: of the first `dims` entries, entry 2i pairs with entry 2i + 1; the pair (a, b) at position p
    becomes (a cos t − b sin t, b cos t + a sin t), t = p · base^(−2i/dims).  Entries beyond dims pass."""
    out = v.clone()
    for i in range(dims // 2):
        t = positions.to(torch.float64) * float(base) ** (-2.0 * i / dims)
        while t.dim() < v.dim() - 1:
            t = t.unsqueeze(-1)
        a, b = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = a * torch.cos(t) - b * torch.sin(t)
        out[..., 2 * i + 1] = b * torch.cos(t) + a * torch.sin(t)
    return out


def causal_softmax_attention(scores, values):
    """scores [H, T, T] (query, key), values [T, H, n] → [T, H, n]; query i sees keys j ≤ i."""
    T = scores.shape[1]
    out = torch.zeros(T, values.shape[1], values.shape[2], dtype=scores.dtype)
    for i in range(T):
        p = torch.softmax(scores[:, i, :i + 1], dim=-1)
        out[i] = torch.einsum("hj,jhn->hn", p, values[:i + 1])
    return out


def latent_attention(h, w, p, m, eps, positions):
    """Queries through a latent; keys and values from a normed latent c, plus one rotated key part r that all heads
    share; a sigmoid gate per head from the same input; the output projection."""
    T, H, dim, vdim, R, C = h.shape[0], m["heads"], m["dim"], m["vdim"], m["rot_dim"], m["kv_rank"]
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, dim + R)
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :C], w[p + "dkv.norm"], eps)
    r = rotate_pairs(down[:, C:], positions, m["rot"]["base"], m["rot"]["dims"])
    qr = rotate_pairs(q[..., dim:], positions, m["rot"]["base"], m["rot"]["dims"])
    k = (c @ w[p + "uk"].T).reshape(T, H, dim)
    v = (c @ w[p + "uv"].T).reshape(T, H, vdim)
    scores = torch.einsum("ihd,jhd->hij", q[..., :dim], k) + torch.einsum("ihd,jd->hij", qr, r)
    out = causal_softmax_attention(scores * m["scale"], v)
    gate = torch.sigmoid(h @ w[p + "g"].T)                          # [T, H]
    return (out * gate[:, :, None]).reshape(T, H * vdim) @ w[p + "o"].T


def mingru_scan(z, cand):
    """S_t = (1 − z_t) · S_(t−1) + z_t · cand_t element by element, S before the first token zero; all S_t."""
    S = torch.zeros_like(z[0])
    out = []
    for t in range(z.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        out.append(S)
    return torch.stack(out)


def mingru(h, w, p):
    z = torch.sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    u = h @ w[p + "x"].T + w[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = mingru_scan(z, cand)
    g = h @ w[p + "g"].T
    return (S * g * torch.sigmoid(g)) @ w[p + "o"].T


def route(z, correction, r):
    """Router logits z [T, E] → chosen experts [T, top] and their weights.  s = softmax(z) over all E; the choice looks
    at s + correction, but only inside the `keep` groups (of `count` equal groups of neighbours) whose largest such
    score is largest; the weights are the chosen s · scale.  Ties go to the lower index."""
    T, E = z.shape
    s = torch.softmax(z, dim=-1)
    choice = s + correction
    count, keep = r["groups"]["count"], r["groups"]["keep"]
    per = E // count
    ids, wts = [], []
    for t in range(T):
        best = [max(choice[t, g * per:(g + 1) * per]) for g in range(count)]
        order = sorted(range(count), key=lambda g: (-float(best[g]), g))[:keep]
        allowed = [e for e in range(E) if e // per in order]
        chosen = sorted(allowed, key=lambda e: (-float(choice[t, e]), e))[:r["top"]]
        ids.append(chosen)
        wts.append([float(s[t, e]) * r["scale"] for e in chosen])
    return ids, wts


def expert(h, w, p):
    a = torch.relu(h @ w[p + "up"].T)
    return (a * a) @ w[p + "down"].T


def routed_ff(h, w, p, ml, margins=None):
    """The last `identity` of the router's outputs stand for experts that return their input."""
    r = ml["router"]
    E, n_id = r["experts"] + r["identity"], r["identity"]
    z = h @ w[p + "router"].T
    ids, wts = route(z, w[p + "correction"], r)
    if margins is not None:
        margins.append(_choice_margin(z, w[p + "correction"], r))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t], wts[t]):
            out[t] += a * (h[t] if e >= E - n_id else expert(h[t:t + 1], w, p + f"e{e}.")[0])
    return out


def _choice_margin(z, correction, r):
    """Per token, how far the choice is from going another way: the smallest gap between a chosen score and the best
    one left out, and between the last kept group and the first dropped, relative to the scores' spread."""
    T, E = z.shape
    s = torch.softmax(z, dim=-1) + correction
    count, keep, top = r["groups"]["count"], r["groups"]["keep"], r["top"]
    per = E // count
    out = []
    for t in range(T):
        best = sorted((float(max(s[t, g * per:(g + 1) * per])) for g in range(count)), reverse=True)
        gap = best[keep - 1] - best[keep] if keep < count else math.inf
        groups = sorted(range(count), key=lambda g: (-float(max(s[t, g * per:(g + 1) * per])), g))[:keep]
        vals = sorted((float(s[t, e]) for e in range(E) if e // per in groups), reverse=True)
        if top < len(vals):
            gap = min(gap, vals[top - 1] - vals[top])
        out.append(gap / max(float(s[t].max() - s[t].min()), 1e-30))
    return torch.tensor(out, dtype=torch.float64)


def schedule(cfg):
    """[(layer, number of the pass that begins with it or None)]: layers start … stop−1 run `times` times in a row."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, k = loop["start"], loop["stop"], loop["times"]
    out = [(i, None) for i in range(a)]
    for t in range(k):
        out += [(i, t if i == a else None) for i in range(a, b)]
    return out + [(i, None) for i in range(b, n)]


def forward(cfg, w, ids, keep_layers=False, margins=None):
    """ids [T] → logits [T, vocab] (and the residual after every layer run, if asked)."""
    w = {k: (v.to(torch.float64) if v.is_floating_point() else v) for k, v in w.items()}
    ids = torch.as_tensor(ids, dtype=torch.long)
    T = ids.shape[0]
    positions = torch.arange(T)
    eps = cfg["norm"]["eps"]
    x = w["embed"][ids] * cfg.get("embedding", {}).get("scale", 1.0)
    kept = []
    for i, begins in schedule(cfg):
        if begins is not None:
            x = x + w["loop.step"][begins]
        layer, p = cfg["layers"][i], f"l{i}."
        h = token_shift(scalar_rms_norm(x, w[p + "norm1"], eps), w[p + "shift"])
        if layer["type"] == "latent_attention":
            x = x + latent_attention(h, w, p + "mix.", layer["mixer"], eps, positions)
        elif layer["type"] == "mingru":
            x = x + mingru(h, w, p + "mix.")
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + routed_ff(scalar_rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"], margins)
        kept.append(x)
    logits = scalar_rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(kept)) if keep_layers else logits


def logits_all_positions(cfg, w, ids):
    return forward(cfg, w, ids)


def decided_prefix(cfg, w, ids, least=0.05):
    """Positions before the first token whose routing (in any layer run) is closer to another outcome than `least`."""
    margins = []
    forward(cfg, w, ids, margins=margins)
    if not margins:
        return len(ids)
    close = torch.stack(margins).min(0).values < least
    idx = torch.nonzero(close)
    return int(idx[0]) if len(idx) else len(ids)


def greedy_generate(cfg, w, prompt, n_new):
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(torch.argmax(forward(cfg, w, ids)[-1])))
    return ids[len(prompt):]
