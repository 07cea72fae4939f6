"""A plain, slow implementation of the Suposun design in float64, one function per mechanism, written from the
design's equations and sharing no code with the package (it reads model folders with the tests' own reader).

Notation: T tokens, width d.  Linear weights are [out, in] and applied as x · Wᵀ.  Everything runs over a whole
sequence from its first token, so there is no cache and no state here: a token's predecessor is simply the token
before it in the list.
"""
from __future__ import annotations

import math

import torch

from plain_gpt2 import read_model_dir  # noqa: F401  (the tests' own reader of config.json + model.safetensors)


def rms_norm(x, w, eps):
    """x / sqrt(mean(x²) + eps) · w."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def one_plus_rms_norm(x, w, eps):
    """The same where w holds the offset from one: the factor is 1 + w."""
    return rms_norm(x, 1.0 + w, eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def bigram_rows(ids, buckets, mul_prev, mul_cur):
    """Row of the bigram table for every token: a hash of (token before, token); the last row for a first token."""
    rows = []
    for t, tok in enumerate(ids):
        rows.append(buckets if t == 0 else (int(ids[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets)
    return torch.tensor(rows, dtype=torch.long)


def embed(cfg, w, ids):
    e = cfg.get("embedding", {})
    x = w["embed"][ids] * e.get("scale", 1.0)
    b = e.get("bigram")
    if b is not None:
        x = x + w["bigram"][bigram_rows(ids.tolist(), b["buckets"], b["mul_prev"], b["mul_cur"])]
    return x


def rotary_frequencies(rot):
    """f_i = base^(−2i/dims) for i < dims/2, and the factor on cos and sin.  With `scaling` (factor, original, fast,
    slow): pairs that turn fewer than `slow` times over `original` positions are slowed by `factor`, pairs that turn more
    than `fast` times are kept, the ones between are blended linearly in the pair's index; cos and sin then grow by
    0.1 · ln(factor) + 1."""
    base, dims = float(rot["base"]), int(rot["dims"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc is None:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def index_of(turns):          # the (real-valued) pair index whose wavelength fits `turns` times into `original`
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(index_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(index_of(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(v, positions, rot, pairing):
    """v [T, heads, n]: the first rot.dims entries of every head are rotated in pairs by position; the rest pass.
    pairing "interleaved": entry 2i with 2i + 1; "half": entry i with i + dims/2."""
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot)
    out = v.clone()
    pos = positions.to(torch.float64)
    for i in range(dims // 2):
        a_i, b_i = (2 * i, 2 * i + 1) if pairing == "interleaved" else (i, i + dims // 2)
        ang = (pos * f[i])[:, None]
        c, s = torch.cos(ang) * mag, torch.sin(ang) * mag
        a, b = v[..., a_i], v[..., b_i]
        out[..., a_i] = a * c - b * s
        out[..., b_i] = b * c + a * s
    return out


def visible(i, j, mask):
    """Whether query position i sees key position j: causal; with a mask also inside the window or among the kept first."""
    if j > i:
        return False
    if mask is None:
        return True
    return (i - j < mask["size"]) or (j < mask.get("keep_first", 0))


def attend(q, k, v, scale, mask=None, softcap=None, sink=None):
    """q [T, H, n], k [T, G, n], v [T, G, m] → [T, H, m].  Scores (q · k) · scale, squashed by cap · tanh(· / cap) where
    there is a cap; softmax over the visible keys, with exp(sink_h) added to the denominator where there are sinks."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, mask)]
            s = (k[js, g] @ q[i, h]) * scale
            if softcap is not None:
                s = softcap * torch.tanh(s / softcap)
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(sink[h] - m) if sink is not None else 0.0)
            out[i, h] = (e / den) @ v[js, g]
    return out


def attention(h, w, p, m, eps, positions):
    """Mixer "attention": values are the projected keys themselves; query/key norm per head with one weight for all
    heads; rotation of neighbouring pairs; a cap on the scores; a window beside which the leading tokens stay visible;
    sinks; a sigmoid gate per head."""
    T, H, G, n = h.shape[0], m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T).view(T, H, n)
    k = (h @ w[p + "k"].T).view(T, G, n)
    v = k
    q = rotate(rms_norm(q, w[p + "q.norm"], eps), positions, m["rot"], "interleaved")
    k = rotate(rms_norm(k, w[p + "k.norm"], eps), positions, m["rot"], "interleaved")
    o = attend(q, k, v, m["scale"], m.get("mask"), m.get("softcap"), w[p + "sink"])
    gate = torch.sigmoid(h @ w[p + "g"].T)                       # [T, H]
    return (o * gate[:, :, None]).reshape(T, -1) @ w[p + "o"].T


def attention_2_keys(h, w, p, m, eps, positions):
    """The keys (normed over the whole projection, rotated by halves) and values that an "attention_2" layer keeps."""
    T, G, n = h.shape[0], m["kv_heads"], m["dim"]
    k = rms_norm(h @ w[p + "k"].T, w[p + "k.norm"], eps).view(T, G, n)
    return rotate(k, positions, m["rot"], "half"), (h @ w[p + "v"].T).view(T, G, m["vdim"])


def attention_2(h, w, p, m, eps, positions, kv):
    """Mixer "attention_2": plain causal softmax attention; kv: the (keys, values) it reads (its own or another layer's)."""
    T, H, n = h.shape[0], m["heads"], m["dim"]
    q = rms_norm(h @ w[p + "q"].T, w[p + "q.norm"], eps).view(T, H, n)
    q = rotate(q, positions, m["rot"], "half")
    o = attend(q, kv[0], kv[1], m["scale"])
    return o.reshape(T, -1) @ w[p + "o"].T


def dense_ff(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def expert(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(h, w, p, ml, margins=None):
    """(chosen experts [T, top], their weights [T, top]): scores sigmoid(W_router h); the choice looks at score +
    correction, the weights are the scores themselves, not renormalized.  Ties go to the lower index."""
    top = ml["router"]["top"]
    s = torch.sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"]
    order = torch.sort(choice, dim=-1, descending=True, stable=True)
    idx = order.indices[:, :top]
    if margins is not None and choice.shape[1] > top:
        margins.append(order.values[:, top - 1] - order.values[:, top])
    return idx, torch.gather(s, 1, idx)


def routed_ff(h, w, p, ml, margins=None):
    idx, wt = route(h, w, p, ml, margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += wt[t, j] * expert(h[t:t + 1], w, p + f"e{e}.", ml["expert"]["limit"])[0]
    return out


def forward(cfg, w, ids, keep_layers=False, margins=None):
    """ids [T] → logits [T, vocab] (and the residual after every layer, if asked)."""
    w = {k: (v.to(torch.float64) if v.is_floating_point() else v) for k, v in w.items()}
    ids = torch.as_tensor(ids, dtype=torch.long)
    positions = torch.arange(ids.shape[0])
    eps = cfg["norm"]["eps"]
    x = embed(cfg, w, ids)
    kept, kv = [], {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            y = attention(x, w, p + "mix.", m, eps, positions)
        elif layer["type"] == "attention_2":
            src = m.get("kv_from")
            if src is None:
                kv[i] = attention_2_keys(x, w, p + "mix.", m, eps, positions)
            y = attention_2(x, w, p + "mix.", m, eps, positions, kv[i if src is None else src])
        else:
            raise ValueError(layer["type"])
        x = x + one_plus_rms_norm(y, w[p + "norm1"], eps) * w[p + "ls1"]
        ml = layer.get("mlp")
        if ml is not None:
            y = dense_ff(x, w, p + "mlp.") if ml["kind"] == "dense" else routed_ff(x, w, p + "mlp.", ml, margins)
            x = x + one_plus_rms_norm(y, w[p + "norm2"], eps) * w[p + "ls2"]
        kept.append(x)
    logits = one_plus_rms_norm(x, w["final.norm"], eps) @ w["embed"].T * cfg.get("logit_scale", 1.0)
    return (logits, torch.stack(kept)) if keep_layers else logits


def logits_all_positions(cfg, w, ids):
    return forward(cfg, w, ids)


def decided_prefix(cfg, w, ids, least=0.02):
    """Positions before the first token whose routing (in any layer) is closer to another outcome than `least`."""
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
