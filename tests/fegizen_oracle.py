"""Plain float64 NumPy implementation of the Fegizen design, one function per mechanism, written from its equations.

It shares nothing with the library: whole sequences at once, explicit loops over positions for everything that has a
window or a state.  `forward(cfg, w, tokens)` returns the logits of every position and the residual stream after every
layer; `make_config` / `make_weights` build small random checkpoints (tests choose their own sizes) and `write_checkpoint`
stores one as config.json + model.safetensors.

Notation: T positions t = 0 .. T-1, width W.  A layer is
    u = N1(x);  x' = x + mixer(u + conv1(u));  v = N2(x');  X = x' + ff(v + conv2(v))
with N a layer norm without bias, conv a causal per-channel convolution, and what the next layer reads is the weighted sum
of the embedding output and all layer results so far (weights '<layer>.dwa').
"""
import json
import math
import os
import struct

import numpy as np


# ---- norms --------------------------------------------------------------------------------------------------------------
def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def rms_norm(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


# ---- input convolution --------------------------------------------------------------------------------------------------
def causal_conv(h, w):
    """conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j), zeros before the start.  h (T, C), w (C, taps)."""
    T, C = h.shape
    taps = w.shape[1]
    out = np.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def with_conv(h, w):
    return h + causal_conv(h, w)


# ---- rotary positions ---------------------------------------------------------------------------------------------------
def rotary_table(rot):
    """Frequencies (dims / 2) and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def corr(turns):
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(corr(float(sc["fast"]))), 0)
    hi = min(math.ceil(corr(float(sc["slow"]))), dims - 1)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, pos, freqs, mag):
    """x (..., dims) at position pos: pairs (2i, 2i+1) turned by pos * freqs[i], cos and sin times mag."""
    out = np.array(x, dtype=np.float64)
    n = len(freqs)
    a = pos * freqs
    c, s = np.cos(a) * mag, np.sin(a) * mag
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out[..., 0:2 * n:2] = u * c - v * s
    out[..., 1:2 * n:2] = v * c + u * s
    return out


# ---- latent attention ---------------------------------------------------------------------------------------------------
def latent_kv(h, m, w, p, eps):
    """The latent c (T, kv_rank) and the rotated shared key part (T, rot_dim) a layer with its own W_dkv caches."""
    r = int(m["kv_rank"])
    freqs, mag = rotary_table(m["rot"])
    ckr = h @ w[p + "dkv"].T
    c = rms_norm(ckr[:, :r], w[p + "dkv.norm"], eps)
    kr = np.stack([rotate_pairs(ckr[t, r:], t, freqs, mag) for t in range(h.shape[0])])
    return c, kr


def latent_attention(h, m, w, p, eps, shared=None):
    """h (T, W) -> (T, W).  shared: (c, kr) of the layer named by kv_from."""
    T = h.shape[0]
    H, dn, dr, dv, r = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    freqs, mag = rotary_table(m["rot"])
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, dn + dr)
    c, kr = shared if shared is not None else latent_kv(h, m, w, p, eps)
    kn = (c @ w[p + "uk"].T).reshape(T, H, dn)
    val = (c @ w[p + "uv"].T).reshape(T, H, dv)
    win, scale = int(m["mask"]["size"]), float(m["scale"])
    out = np.zeros((T, H, dv))
    for t in range(T):
        lo = max(0, t - win + 1)
        qr = rotate_pairs(q[t, :, dn:], t, freqs, mag)
        for hh in range(H):
            s = (kn[lo:t + 1, hh] @ q[t, hh, :dn] + kr[lo:t + 1] @ qr[hh]) * scale
            e = np.exp(s - s.max())
            out[t, hh] = (e / e.sum()) @ val[lo:t + 1, hh]
    gate = 1.0 / (1.0 + np.exp(-(h @ w[p + "g"].T)))
    return (out.reshape(T, H * dv) * gate) @ w[p + "o"].T


# ---- gated linear attention ---------------------------------------------------------------------------------------------
def gla_scan(q, k, v, alpha):
    """Per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k, alpha (T, H, D), v (T, H, P)."""
    T, H, D = q.shape
    P = v.shape[2]
    S = np.zeros((H, D, P))
    o = np.zeros((T, H, P))
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdp,hd->hp", S, q[t])
    return o


def gla(h, m, w, p, eps):
    T = h.shape[0]
    H, D, P, tau = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["tau"])
    q = (h @ w[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, D)
    v = (h @ w[p + "v"].T).reshape(T, H, P)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = (1.0 / (1.0 + np.exp(-z))) ** (1.0 / tau)
    o = gla_scan(q, k, v, alpha.reshape(T, H, D))
    o = rms_norm(o, w[p + "norm"], eps).reshape(T, H * P)
    g = h @ w[p + "g"].T
    return (o * (g / (1.0 + np.exp(-g)))) @ w[p + "o"].T


# ---- feed-forward -------------------------------------------------------------------------------------------------------
def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + np.exp(-z))


def glu(h, w, p, act):
    return (act(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, f, w, p):
    """Chosen experts (T, top) and their weights.  Indices >= experts are identity experts."""
    r = f["router"]
    z = h @ w[p + "router"].T
    e = np.exp(z - z.max(-1, keepdims=True))
    s = e / e.sum(-1, keepdims=True)
    choice = s + w[p + "correction"] if (p + "correction") in w else s
    top = int(r["top"])
    ids = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    ws = np.take_along_axis(s, ids, -1)
    ws = ws / (ws.sum(-1, keepdims=True) + 1e-20) * float(r.get("scale", 1.0))
    return ids, ws


def moe(h, f, w, p):
    E = int(f["router"]["experts"])
    ids, ws = route(h, f, w, p)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(ids[t], ws[t]):
            out[t] += wt * (h[t] if e >= E else glu(h[t:t + 1], w, "%se%d." % (p, e), silu)[0])
    if f.get("shared"):
        out += glu(h, w, p + "shared.", silu)
    return out


def feed_forward(h, f, w, p):
    return glu(h, w, p, gelu_tanh) if f["kind"] == "dense" else moe(h, f, w, p)


# ---- the model ----------------------------------------------------------------------------------------------------------
def forward(cfg, w, tokens):
    """-> logits (T, vocab), residual stream after every layer (L, T, W); all float64."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    eps, taps = float(cfg["norm"]["eps"]), int(cfg["canon"]["taps"])
    x = w["embed"][np.asarray(tokens)] * float(cfg["embedding"]["scale"])
    results, after, latents = [x], [], {}
    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        assert w[p + "canon1"].shape[1] == taps
        u = with_conv(layer_norm(x, w[p + "norm1"], eps), w[p + "canon1"])
        if L["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_kv(u, m, w, p + "mix.", eps)
            y = latent_attention(u, m, w, p + "mix.", eps, latents[i if src is None else int(src)])
        elif L["type"] in ("gla", "gla_2"):
            y = gla(u, m, w, p + "mix.", eps)
        else:
            raise ValueError(L["type"])
        x = x + y
        if L.get("mlp"):
            u = with_conv(layer_norm(x, w[p + "norm2"], eps), w[p + "canon2"])
            x = x + feed_forward(u, L["mlp"], w, p + "mlp.")
        results.append(x)
        x = sum(w[p + "dwa"][j] * results[j] for j in range(i + 2))
        after.append(x)
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T * float(cfg["logit_scale"])
    return logits, np.stack(after)


def greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(forward(cfg, w, toks)[0][-1])))
    return toks[len(prompt):]


# ---- small random checkpoints -------------------------------------------------------------------------------------------
def bf16_round(a):
    """float -> nearest bfloat16 (ties to even), as float32."""
    u = np.asarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def latent_mixer(heads=4, dim=16, rot_dim=8, vdim=16, kv_rank=24, q_rank=32, window=12, base=10000.0, scaling=True, kv_from=None, scale=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = {"factor": 8.0, "fast": 24.0, "original": 64, "slow": 2.0}
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "mask": {"size": window}, "rot": rot,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def gla_mixer(heads=2, dim=16, vdim=24, tau=8.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def dense_mlp(ff=48):
    return {"kind": "dense", "ff": ff}


def moe_mlp(ff=24, experts=5, identity=2, top=2, scale=1.5, shared=40):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def make_config(layers, width=48, vocab=96, taps=3, eps=1e-5, embed_scale=4.0, logit_scale=0.5):
    """layers: list of (type, mixer dict, mlp dict or None)."""
    return {"architecture": "Fegizen", "canon": {"taps": taps}, "embedding": {"scale": embed_scale},
            "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in layers], "logit_scale": logit_scale, "norm": {"eps": eps}, "vocab": vocab,
            "width": width}


def make_weights(cfg, seed=0, a_rank=6, router_gain=1.0):
    """Random weights, rounded to bfloat16 values (float32 arrays)."""
    rng = np.random.default_rng(seed)
    W, V, taps = cfg["width"], cfg["vocab"], cfg["canon"]["taps"]
    w = {}

    def lin(name, out, inp, gain=1.0):
        w[name] = rng.standard_normal((out, inp)) * gain / math.sqrt(inp)

    def ones(name, n, spread=0.2):
        w[name] = 1.0 + spread * rng.standard_normal(n)

    w["embed"] = rng.standard_normal((V, W)) / cfg["embedding"]["scale"]
    for i, L in enumerate(cfg["layers"]):
        p, m, f = "l%d." % i, L["mixer"], L["mlp"]
        ones(p + "norm1", W)
        w[p + "canon1"] = 0.3 * rng.standard_normal((W, taps))
        q = p + "mix."
        if L["type"] == "latent_attention":
            H, dn, dr, dv, r, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            lin(q + "dq", qr, W), ones(q + "dq.norm", qr), lin(q + "uq", H * (dn + dr), qr, 2.0)
            if m.get("kv_from") is None:
                lin(q + "dkv", r + dr, W, 2.0), ones(q + "dkv.norm", r)
            lin(q + "uk", H * dn, r, 2.0), lin(q + "uv", H * dv, r), lin(q + "g", H * dv, W), lin(q + "o", W, H * dv)
        else:
            H, D, P = m["heads"], m["dim"], m["vdim"]
            lin(q + "q", H * D, W, 2.0), lin(q + "k", H * D, W), lin(q + "v", H * P, W), lin(q + "g", H * P, W), lin(q + "o", W, H * P)
            ones(q + "norm", P), lin(q + "a1", a_rank, W), lin(q + "a2", H * D, a_rank, 2.0)
            w[q + "a2.b"] = 2.0 + rng.standard_normal(H * D)
        if f:
            ones(p + "norm2", W)
            w[p + "canon2"] = 0.3 * rng.standard_normal((W, taps))
            q = p + "mlp."
            if f["kind"] == "dense":
                lin(q + "gate", f["ff"], W), lin(q + "up", f["ff"], W), lin(q + "down", W, f["ff"])
            else:
                r = f["router"]
                n_all = r["experts"] + r.get("identity", 0)
                for e in range(r["experts"]):
                    lin("%se%d.gate" % (q, e), f["expert"]["ff"], W), lin("%se%d.up" % (q, e), f["expert"]["ff"], W)
                    lin("%se%d.down" % (q, e), W, f["expert"]["ff"])
                lin(q + "router", n_all, W, router_gain)
                w[q + "correction"] = 0.05 * rng.standard_normal(n_all)
                if f.get("shared"):
                    lin(q + "shared.gate", f["shared"]["ff"], W), lin(q + "shared.up", f["shared"]["ff"], W), lin(q + "shared.down", W, f["shared"]["ff"])
        d = rng.standard_normal(i + 2) * 0.2
        d[-1] += 1.0
        w[p + "dwa"] = d
    ones("final.norm", W)
    lin("head", V, W)
    return {k: bf16_round(v) for k, v in w.items()}


def write_checkpoint(folder, cfg, w):
    """config.json + model.safetensors (bfloat16 tensors)."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    head, blobs, at = {}, [], 0
    for name, a in w.items():
        b = (np.asarray(a, dtype=np.float32).view(np.uint32) >> 16).astype("<u2").tobytes()
        head[name] = {"dtype": "BF16", "shape": list(np.shape(a)), "data_offsets": [at, at + len(b)]}
        blobs.append(b)
        at += len(b)
    hj = json.dumps(head).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
