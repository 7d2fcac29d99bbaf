"""Plain float64 NumPy implementation of the Kiduvik design, one function per mechanism, written from its equations.

It shares nothing with the library: whole sequences at once, explicit loops over positions and heads, keys and values per
head as the equations give them.  `forward(cfg, w, tokens)` returns the logits of every position and the residual stream
after every layer; `make_config` / `make_weights` build small random checkpoints (tests choose their own sizes) and
`write_checkpoint` stores one as config.json + model.safetensors.

Notation: T positions t = 0 .. T-1, width W, eps = norm.eps, rms(z) = z / sqrt(mean(z^2) + eps).  A layer is
    x' = x + rms(mixer(rms(x) n1)) n1b;   x'' = x' + rms(ff(rms(x') n2)) n2b;   X = x'' + rms(P (gelu_tanh(G x'') * e)) ns
with e the layer's slice of a second embedding of the token ("token side input").
"""
import json
import math
import os
import struct

import numpy as np


# ---- norms and activations ----------------------------------------------------------------------------------------------
def rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


_erf = np.vectorize(math.erf, otypes=[np.float64])


def gelu_erf(z):
    return 0.5 * z * (1.0 + _erf(z / math.sqrt(2.0)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


# ---- rotary positions, half-split pairs ---------------------------------------------------------------------------------
def rotary_table(rot):
    """Frequencies (dims / 2) and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def where(turns):
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x, pos, freqs, mag):
    """x (..., >= dims) at position pos: channel i pairs with channel i + dims / 2; the rest passes."""
    n = len(freqs)
    out = np.array(x, dtype=np.float64)
    a = pos * freqs
    c, s = np.cos(a) * mag, np.sin(a) * mag
    u, v = x[..., :n], x[..., n:2 * n]
    out[..., :n] = u * c - v * s
    out[..., n:2 * n] = v * c + u * s
    return out


# ---- latent attention with a sink ---------------------------------------------------------------------------------------
def latent_rows(h, m, w, p, eps):
    """What a layer with its own W_dkv caches: the latent c (T, kv_rank) and the rotated shared key part (T, rot_dim)."""
    r = int(m["kv_rank"])
    freqs, mag = rotary_table(m["rot"])
    z = h @ w[p + "dkv"].T
    c = rms_norm(z[:, :r], w[p + "dkv.norm"], eps)
    kr = np.stack([rotate_half(z[t, r:], t, freqs, mag) for t in range(h.shape[0])])
    return c, kr


def softmax_with_sink(s, sink):
    """Weights over the keys when the denominator also holds exp(sink) (no key, no value; sink None: plain softmax)."""
    top = s.max() if sink is None else max(s.max(), sink)
    e = np.exp(s - top)
    return e / (e.sum() + (0.0 if sink is None else math.exp(sink - top)))


def latent_attention(h, m, w, p, eps, shared=None):
    """h (T, W) -> (T, W), causal.  shared: (c, kr) of the layer that kv_from names."""
    T = h.shape[0]
    H, dn, dr, dv = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
    freqs, mag = rotary_table(m["rot"])
    q = (h @ w[p + "q"].T).reshape(T, H, dn + dr)
    c, kr = shared if shared is not None else latent_rows(h, m, w, p, eps)
    ku = (c @ w[p + "uk"].T).reshape(T, H, dn)
    val = (c @ w[p + "uv"].T).reshape(T, H, dv)
    scale = float(m["scale"])
    out = np.zeros((T, H, dv))
    for t in range(T):
        qr = rotate_half(q[t, :, dn:], t, freqs, mag)
        for a in range(H):
            s = (ku[:t + 1, a] @ q[t, a, :dn] + kr[:t + 1] @ qr[a]) * scale
            out[t, a] = softmax_with_sink(s, float(w[p + "sink"][a])) @ val[:t + 1, a]
    return out.reshape(T, H * dv) @ w[p + "o"].T


# ---- differential attention over a window with kept first tokens ------------------------------------------------------
def visible(i, j, size, keep_first):
    return j <= i and (i - j < size or j < keep_first)


def diff_lambda(m, w, p):
    return math.exp(float(w[p + "lq1"] @ w[p + "lk1"])) - math.exp(float(w[p + "lq2"] @ w[p + "lk2"])) + float(m["diff"])


def diff_attention(h, m, w, p, eps):
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    size, keep = int(m["mask"]["size"]), int(m["mask"]["keep_first"])
    freqs, mag = rotary_table(m["rot"])
    q = (h @ w[p + "q"].T).reshape(T, H, 2, d)
    k = (h @ w[p + "k"].T).reshape(T, G, 2, d)
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    for t in range(T):
        q[t] = rotate_half(q[t], t, freqs, mag)
        k[t] = rotate_half(k[t], t, freqs, mag)
    lam, diff, scale = diff_lambda(m, w, p), float(m["diff"]), float(m["scale"])
    gate = sigmoid(h @ w[p + "g"].T)  # (T, H)
    out = np.zeros((T, H, dv))
    for t in range(T):
        js = [j for j in range(t + 1) if visible(t, j, size, keep)]
        for a in range(H):
            g = a // (H // G)
            maps = []
            for r in range(2):
                s = (k[js, g, r] @ q[t, a, r]) * scale
                maps.append(softmax_with_sink(s, None) @ v[js, g])
            o = maps[0] - lam * maps[1]
            out[t, a] = rms(o, eps) * (1.0 - diff) * gate[t, a]
    return out.reshape(T, H * dv) @ w[p + "o"].T


# ---- feed-forward and the token side input ----------------------------------------------------------------------------
def dense_ff(h, w, p):
    return gelu_erf(h @ w[p + "up"].T) @ w[p + "down"].T


def token_side(x, tokens, layer, cfg, w, eps):
    d = int(cfg["token_side"]["dim"])
    p = "l%d.side." % layer
    e = w["side.embed"][tokens][:, layer * d:(layer + 1) * d]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return rms_norm(y, w[p + "norm"], eps)


# ---- the model ----------------------------------------------------------------------------------------------------------
def forward(cfg, w, tokens):
    """Logits (T, vocab) and the residual stream after every layer (layers, T, W)."""
    tokens = np.asarray(tokens)
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][tokens] + w["pos"][:len(tokens)]
    caches, after = {}, []
    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        h = rms_norm(x, w[p + "norm1"], eps)
        if L["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                caches[i] = latent_rows(h, m, w, p + "mix.", eps)
            y = latent_attention(h, m, w, p + "mix.", eps, caches[i if src is None else src])
        elif L["type"] == "attention":
            y = diff_attention(h, m, w, p + "mix.", eps)
        else:
            raise ValueError(L["type"])
        x = x + rms_norm(y, w[p + "norm1b"], eps)
        if L.get("mlp"):
            x = x + rms_norm(dense_ff(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp."), w[p + "norm2b"], eps)
        if cfg.get("token_side"):
            x = x + token_side(x, tokens, i, cfg, w, eps)
        after.append(x.copy())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T, np.stack(after)


def greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(forward(cfg, w, toks)[0][-1])))
    return toks[len(prompt):]


def bf16_round(a):
    u = np.asarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.float64)


# ---- small random checkpoints -------------------------------------------------------------------------------------------
def latent_mixer(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, base=10000.0, kv_from=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "rot": {"dims": rot_dim, "base": base},
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def diff_mixer(heads=4, kv_heads=2, dim=16, vdim=24, size=10, keep_first=2, rot_dims=8, base=10000.0, scaling=True, diff=0.3, scale=None):
    rot = {"dims": rot_dims, "base": base}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
                                           "mask": {"size": size, "keep_first": keep_first}, "rot": rot,
                                           "scale": scale if scale is not None else dim ** -0.5}}


def make_config(layers, width=48, vocab=96, ff=80, side=8, eps=1e-5, max_positions=512):
    out = []
    for L in layers:
        L = dict(L)
        L.setdefault("mlp", {"kind": "dense", "ff": ff} if ff else None)
        out.append(L)
    cfg = {"architecture": "Kiduvik", "width": width, "vocab": vocab, "max_positions": max_positions, "norm": {"eps": eps}, "layers": out}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


def make_weights(cfg, seed=0, gain=1.0):
    """Random weights, rounded to bf16 (what a checkpoint stores)."""
    rng = np.random.default_rng(seed)
    W, V = cfg["width"], cfg["vocab"]
    w = {}

    def mat(name, o, i, g=1.0):
        w[name] = bf16_round(rng.standard_normal((o, i)) * g * gain / math.sqrt(i))

    def vec(name, n, around=1.0, spread=0.2):
        w[name] = bf16_round(around + spread * rng.standard_normal(n))

    w["embed"] = bf16_round(rng.standard_normal((V, W)))
    w["pos"] = bf16_round(0.5 * rng.standard_normal((cfg["max_positions"], W)))
    side = cfg.get("token_side")
    if side:
        w["side.embed"] = bf16_round(rng.standard_normal((V, side["dim"] * len(cfg["layers"]))))
    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        for n in ("norm1", "norm2", "norm1b", "norm2b"):
            if n.startswith("norm2") and not L.get("mlp"):
                continue
            vec(p + n, W)
        q = p + "mix."
        if L["type"] == "latent_attention":
            H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            mat(q + "q", H * (dn + dr), W, 2.0)
            if m.get("kv_from") is None:
                mat(q + "dkv", r + dr, W, 2.0)
                vec(q + "dkv.norm", r)
            mat(q + "uk", H * dn, r, 2.0)
            mat(q + "uv", H * dv, r)
            vec(q + "sink", H, 0.5, 1.0)
            mat(q + "o", W, H * dv)
        else:
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            mat(q + "q", H * 2 * d, W, 2.0)
            mat(q + "k", G * 2 * d, W, 2.0)
            mat(q + "v", G * dv, W)
            vec(q + "q.norm", d, 1.5)
            vec(q + "k.norm", d, 1.5)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                vec(q + n, d, 0.0, 0.25)
            mat(q + "g", H, W, 2.0)
            mat(q + "o", W, H * dv)
        if L.get("mlp"):
            mat(p + "mlp.up", L["mlp"]["ff"], W)
            mat(p + "mlp.down", W, L["mlp"]["ff"])
        if side:
            mat(p + "side.gate", side["dim"], W, 2.0)
            mat(p + "side.proj", W, side["dim"])
            vec(p + "side.norm", W, 0.5)
    vec("final.norm", W)
    mat("head", V, W)
    return w


def write_checkpoint(folder, cfg, w):
    """config.json + model.safetensors (bf16)."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    for name, a in w.items():
        if np.size(a) == 0:      # a head part of size zero has no tensor
            continue
        b = (np.asarray(a, dtype=np.float32).view(np.uint32) >> 16).astype("<u2").tobytes()
        header[name] = {"dtype": "BF16", "shape": list(np.shape(a)), "data_offsets": [at, at + len(b)]}
        blobs.append(b)
        at += len(b)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
