"""-m gpu: the Kiduvik design on the layered executor against the plain float64 statement in kiduvik_oracle.py.

The new row ops alone (device arrays through the C ABI): per-head q / k norm + half-split rotation + cache append with the
kept-first buffers; the softmax sink in every attention kernel, with a sink that outweighs all keys and one that is negligible;
the window with kept first tokens and two maps over shared values, with crafted queries that single out one key at every edge
(oldest inside the window, newest outside, last kept, first not kept, position 0, the query itself) over wrapping rings in
portions of 1 to whole; a far key among hundreds of latent rows; the maps' combination; the exact GELU; the token side input.
Then small models with random weights whose sizes differ from layer to layer: every mechanism through the residual after its
layer; whole prompts against token-by-token decoding and portions down to two tokens; caches given back and used again; long
decoding over a wrapping ring; tensor-core prompt routes and serving precision; greedy generation through the library's entry
points, the command line and the trace runner.
"""
import ctypes as C
import json
import math
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

import kiduvik_oracle as O
from yalm_b200 import api

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32_TOL = 3e-4
vp, i32, f32 = C.c_void_p, C.c_int, C.c_float


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.ascontiguousarray(a), dtype=dtype).cuda().contiguous()


def ptr(t):
    return vp(t.data_ptr()) if t is not None else None


def ok(rc, what):
    torch.cuda.synchronize()
    assert rc == 0, "%s returned %d" % (what, rc)


def close_enough(got, want, tol=F32_TOL):
    scale = max(1.0, float(np.abs(want).max()))
    err = float(np.abs(np.asarray(got, np.float64) - want).max())
    assert err <= tol * scale, f"max |delta| {err:.3e} > {tol * scale:.3e}"


def portions(T, sizes):
    at, k = 0, 0
    while at < T:
        n = min(sizes[k % len(sizes)], T - at)
        yield at, n
        at, k = at + n, k + 1


def L():
    lib = api.lib()
    lib.yalm_attn_window_pool_workspace.restype = C.c_size_t
    return lib


def workspace(dv):
    return torch.zeros(int(L().yalm_attn_window_pool_workspace(dv)), dtype=torch.float32, device="cuda")


# ---- per-head norm, rotation, append -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("cache_f32", [1, 0])
@pytest.mark.parametrize("dk,dv,rot_dims,scaling", [(16, 24, 8, True), (48, 40, 48, False), (20, 8, 0, False), (72, 96, 24, True)])
def test_head_norm_rotation_append(dk, dv, rot_dims, scaling, cache_f32):
    rng = np.random.default_rng(dk)
    nq, nk, nv, T, ring, keep, eps = 6, 4, 2, 23, 16, 3, 1e-5
    ld = nq * dk + nk * dk + nv * dv + 5
    o_q, o_k, o_v = 2, 2 + nq * dk, 2 + (nq + nk) * dk
    P = rng.standard_normal((T, ld))
    qw, kw = 1 + 0.3 * rng.standard_normal(dk), 1 + 0.3 * rng.standard_normal(dk)
    rot = {"dims": rot_dims, "base": 50.0}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}
    fr, mag = O.rotary_table(rot) if rot_dims else (np.zeros(0), 1.0)
    want_q = np.zeros((T, nq, dk))
    want_k = np.zeros((T, nk, dk))
    for t in range(T):
        want_q[t] = O.rotate_half(O.rms_norm(P[t, o_q:o_q + nq * dk].reshape(nq, dk), qw, eps), t, fr, mag)
        want_k[t] = O.rotate_half(O.rms_norm(P[t, o_k:o_k + nk * dk].reshape(nk, dk), kw, eps), t, fr, mag)
    want_v = P[:, o_v:o_v + nv * dv].reshape(T, nv, dv)
    ct = torch.float32 if cache_f32 else torch.bfloat16
    Pd, kr, vr = dev(P), torch.zeros((nk, ring, dk), dtype=ct, device="cuda"), torch.zeros((nv, ring, dv), dtype=ct, device="cuda")
    kf, vf = torch.zeros((nk, keep, dk), device="cuda"), torch.zeros((nv, keep, dv), device="cuda")
    frd, qwd, kwd = dev(fr) if rot_dims else None, dev(qw), dev(kw)
    for at, n in portions(T, [1, 2, 7, 5]):
        ok(L().yalm_head_norm_rope_append_rows(ptr(Pd[at:]), ld, o_q, o_k, o_v, nq, nk, nv, dk, dv, ptr(qwd), ptr(kwd), ptr(frd), f32(mag), rot_dims, 0,
                                               f32(eps), ptr(kr), ptr(vr), ring, ptr(kf), ptr(vf), keep, cache_f32, n, at, None, None), "head_norm_rope_append_rows")
    tol = F32_TOL if cache_f32 else 1e-2
    close_enough(Pd.cpu().numpy()[:, o_q:o_q + nq * dk].reshape(T, nq, dk), want_q)
    last = np.arange(T - ring, T)                                 # the ring holds the last `ring` positions at slot p % ring
    close_enough(kr.float().cpu().numpy()[:, last % ring], want_k[last].transpose(1, 0, 2), tol)
    close_enough(vr.float().cpu().numpy()[:, last % ring], want_v[last].transpose(1, 0, 2), tol)
    close_enough(kf.cpu().numpy(), want_k[:keep].transpose(1, 0, 2), tol)   # the first tokens survive the ring's wrap
    close_enough(vf.cpu().numpy(), want_v[:keep].transpose(1, 0, 2), tol)


def test_interleaved_pairs_are_the_other_layout():
    dk, T = 8, 3
    x = np.random.default_rng(0).standard_normal((T, dk))
    fr, _ = O.rotary_table({"dims": dk, "base": 10.0})
    Pd = dev(np.concatenate([x, x, np.zeros((T, 4))], 1))
    kr, vr = torch.zeros((1, 4, dk), device="cuda"), torch.zeros((1, 4, 4), device="cuda")
    frd = dev(fr)
    ok(L().yalm_head_norm_rope_append_rows(ptr(Pd), 2 * dk + 4, 0, dk, 2 * dk, 1, 1, 1, dk, 4, None, None, ptr(frd), f32(1.0), dk, 1, f32(1e-5), ptr(kr), ptr(vr), 4,
                                           None, None, 0, 1, T, 0, None, None), "interleaved")
    got = Pd.cpu().numpy()[:, :dk]
    for t in range(T):
        perm = np.concatenate([np.arange(0, dk, 2), np.arange(1, dk, 2)])       # pairs (2 i, 2 i + 1) seen as (i, i + half)
        want = np.empty(dk)
        want[perm] = O.rotate_half(x[t][perm], t, fr, 1.0)
        close_enough(got[t], want)


# ---- attention: sink, window with kept first tokens, shared values ----------------------------------------------------------------
def plain_attention(q, k, v, scale, size, keep, sink, v_heads):
    """q (T, H, d), k (T, G, d), v (T, Gv, dv): head h reads key head h // (H / G) and value head (that) % Gv."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for t in range(T):
        js = [j for j in range(t + 1) if O.visible(t, j, size if size > 0 else T + 1, keep)]
        for h in range(H):
            g = h // (H // G)
            p = O.softmax_with_sink((k[js, g] @ q[t, h]) * scale, None if sink is None else float(sink[h]))
            out[t, h] = p @ v[js, g % v_heads]
    return out


def run_window_attention(q, k, v, scale, size, keep, sink, v_heads, ring, cache_f32, sizes, mma=False):
    T, H, d = q.shape
    G, Gv, dv = k.shape[1], v.shape[1], v.shape[2]
    ld = (H + G) * d + Gv * dv
    Pd = dev(np.concatenate([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1))
    ct = torch.float32 if cache_f32 else torch.bfloat16
    kr, vr = torch.zeros((G, ring, d), dtype=ct, device="cuda"), torch.zeros((Gv, ring, dv), dtype=ct, device="cuda")
    kf = torch.zeros((G, max(keep, 1), d), device="cuda")
    vf = torch.zeros((Gv, max(keep, 1), dv), device="cuda")
    out = torch.zeros((T, H * dv), device="cuda")
    ws = workspace(dv)
    sk = dev(sink) if sink is not None else None
    for at, n in portions(T, sizes):
        ok(L().yalm_head_norm_rope_append_rows(ptr(Pd[at:]), ld, 0, H * d, (H + G) * d, H, G, Gv, d, dv, None, None, None, f32(1.0), 0, 0, f32(1e-5), ptr(kr), ptr(vr), ring,
                                               ptr(kf), ptr(vf), keep, cache_f32, n, at, None, None), "append")
        if mma:
            ok(L().yalm_attn_window_pool_mma_sink(ptr(out[at:]), H * dv, ptr(Pd[at:]), ld, ptr(kr), ptr(vr), ptr(kf) if keep else None, ptr(vf) if keep else None, n, H, G, d, dv,
                                                  ring, keep, size, 1 if keep else 0, f32(scale), at, None, ptr(sk), Gv, None), "attn_window_pool_mma_sink")
        else:
            ok(L().yalm_attn_window_pool_sink(ptr(out[at:]), H * dv, ptr(Pd[at:]), ld, ptr(kr), d, ptr(vr), dv, ptr(kf) if keep else None, ptr(vf) if keep else None, ptr(ws), n,
                                              H, G, d, dv, ring, keep, size, 1 if keep else 0, f32(scale), cache_f32, T, at, None, ptr(sk), Gv, None), "attn_window_pool_sink")
    return out.cpu().numpy().reshape(T, H, dv)


def crafted(T, H, G, d, dv, Gv, size, keep, seed=0):
    """Small random q, k, v; row t's head h % 6 asks, with a score near 40, for one key at an edge of what it may see."""
    rng = np.random.default_rng(seed)
    q, k, v = 0.3 * rng.standard_normal((T, H, d)), 0.3 * rng.standard_normal((T, G, d)), rng.standard_normal((T, Gv, dv))
    for t in range(T):
        edges = [t - size + 1, t - size, keep - 1, keep, 0, t]        # oldest inside, newest outside, last kept, first not kept, first, itself
        for h in range(H):
            j = edges[(h + t) % 6]
            if 0 <= j <= t:
                g = h // (H // G)
                u = k[j, g] / np.linalg.norm(k[j, g])
                q[t, h] = 40.0 * u / np.linalg.norm(k[j, g])
    return q, k, v


@pytest.mark.parametrize("cache_f32", [1, 0])
@pytest.mark.parametrize("sizes", [[1], [2], [7, 1, 3], [64]])
@pytest.mark.parametrize("d,dv,H,G,Gv", [(16, 24, 8, 4, 2), (48, 40, 6, 2, 1), (32, 64, 4, 4, 2)])
def test_window_edges_kept_first_tokens_and_shared_values(d, dv, H, G, Gv, sizes, cache_f32):
    T, size, keep = 61, 9, 3
    ring = 16 + max(sizes)
    q, k, v = crafted(T, H, G, d, dv, Gv, size, keep, seed=d)
    if not cache_f32:
        q, k, v = O.bf16_round(q), O.bf16_round(k), O.bf16_round(v)
    want = plain_attention(q, k, v, 1.0, size, keep, None, Gv)
    got = run_window_attention(q, k, v, 1.0, size, keep, None, Gv, ring, cache_f32, sizes)
    close_enough(got, want, F32_TOL if cache_f32 else 2e-3)
    # the crafted queries make every edge count: a window one key longer or shorter, or one kept token more or fewer, is another result
    for other in (plain_attention(q, k, v, 1.0, size + 1, keep, None, Gv), plain_attention(q, k, v, 1.0, size - 1, keep, None, Gv),
                  plain_attention(q, k, v, 1.0, size, keep + 1, None, Gv), plain_attention(q, k, v, 1.0, size, keep - 1, None, Gv)):
        assert np.abs(other - want).max() > 0.1


@pytest.mark.parametrize("keep", [0, 5])
def test_window_edges_on_the_tensor_cores(keep):
    T, size, d, dv, H, G, Gv = 150, 40, 64, 32, 4, 2, 1
    q, k, v = crafted(T, H, G, d, dv, Gv, size, keep, seed=2)
    q, k, v = O.bf16_round(q), O.bf16_round(k), O.bf16_round(v)
    sink = np.array([-1.0, 0.5, 30.0, 2.0])
    want = plain_attention(q, k, v, 0.5, size, keep, sink, Gv)
    for sizes in ([150], [70, 33, 47]):
        got = run_window_attention(q, k, v, 0.5, size, keep, sink, Gv, 256, 0, sizes, mma=True)
        close_enough(got, want, 1e-2)


@pytest.mark.parametrize("cache_f32", [1, 0])
def test_sink_in_the_denominator(cache_f32):
    """A sink far above every score leaves almost nothing for the keys, one far below changes nothing, one near them takes its share."""
    T, H, d, dv = 70, 3, 16, 24
    rng = np.random.default_rng(5)
    q, k, v = O.bf16_round(rng.standard_normal((T, H, d))), O.bf16_round(rng.standard_normal((T, 1, d))), O.bf16_round(rng.standard_normal((T, 1, dv)))
    sink = np.array([60.0, -60.0, 0.7])
    want = plain_attention(q, k, v, 0.25, 0, 0, sink, 1)
    none = plain_attention(q, k, v, 0.25, 0, 0, None, 1)
    assert np.abs(want[:, 0]).max() < 1e-6 and np.abs(want[:, 1] - none[:, 1]).max() < 1e-12 and np.abs(want[:, 2] - none[:, 2]).max() > 0.05
    for sizes in ([1], [5, 2], [70]):          # decode rows split the keys and merge: the sink joins once, at the end
        got = run_window_attention(q, k, v, 0.25, 0, 0, sink, 1, 128, cache_f32, sizes)
        close_enough(got, want, F32_TOL if cache_f32 else 2e-3)


@pytest.mark.parametrize("sizes", [[1], [3, 2], [700]])
def test_latent_rows_far_key_and_sink(sizes):
    """700 cached rows shared by all heads, values inside the rows; one head asks for position 3 from everywhere, one has a heavy sink."""
    T, H, dk, dv = 700, 4, 48, 32
    rng = np.random.default_rng(6)
    rows = O.bf16_round(0.3 * rng.standard_normal((T, dk)))
    q = 0.3 * rng.standard_normal((T, H, dk))
    q[:, 0] = 40.0 * rows[3] / (rows[3] @ rows[3])
    sink = np.array([0.0, 50.0, -3.0, 1.0])
    want = np.zeros((T, H, dv))
    for t in range(T):
        for h in range(H):
            want[t, h] = O.softmax_with_sink(rows[:t + 1] @ q[t, h], float(sink[h])) @ rows[:t + 1, :dv]
    assert np.abs(want[100:, 0] - rows[3, :dv]).max() < 0.05       # the far key carries head 0
    R = dev(rows, torch.bfloat16)
    Q, out, ws, sk = dev(q.reshape(T, -1)), torch.zeros((T, H * dv), device="cuda"), workspace(dv), dev(sink)
    for at, n in portions(T, sizes):
        if at > 40 and at < 650 and sizes != [700]:
            continue                                                # decode-sized calls: the start, and the far end
        ok(L().yalm_attn_latent_rows_sink(ptr(out[at:]), H * dv, ptr(Q[at:]), H * dk, ptr(R), dk, ptr(ws), n, H, dk, dv, T, 0, f32(1.0), T, at, None, ptr(sk), None),
           "attn_latent_rows_sink")
    got = out.cpu().numpy().reshape(T, H, dv)
    done = [t for at, n in portions(T, sizes) if not (at > 40 and at < 650 and sizes != [700]) for t in range(at, at + n)]
    close_enough(got[done], want[done], 2e-3)


@pytest.mark.parametrize("H,dk,dv,window,nsplit", [(6, 96, 64, 0, 1), (6, 96, 64, 0, 7), (20, 80, 64, 37, 3), (16, 576, 512, 0, 64), (7, 96, 64, 0, 128), (3, 272, 256, 130, 2), (33, 144, 128, 0, 5)])
def test_latent_rows_on_the_tensor_cores(H, dk, dv, window, nsplit):
    """Decode-sized calls with the heads as the M tile: head counts below, at and above 16, key splits from one to more than there are
    tiles, a window over a wrapping ring, crafted queries at the window's edges, position 0, the far start, and a sink per head."""
    T, ring = 300, 300 if window == 0 else 192
    rng = np.random.default_rng(H + dk)
    rows = O.bf16_round(0.3 * rng.standard_normal((T, dk)))
    q = O.bf16_round(0.1 * rng.standard_normal((T, H, dk)))
    size = window if window > 0 else T + 1
    for t in range(T):
        for h in range(H):
            j = [t - size + 1, t - size, 0, t, 3, t - 64][(h + t) % 6]      # oldest inside, newest outside, first, itself, far start, a tile back
            if 0 <= j <= t:
                q[t, h] = O.bf16_round(30.0 * rows[j] / (rows[j] @ rows[j]))
    sink = rng.standard_normal(H) * 3.0
    want = np.zeros((T, H, dv))
    for t in range(T):
        lo = max(0, t - size + 1)
        for h in range(H):
            want[t, h] = O.softmax_with_sink(rows[lo:t + 1] @ q[t, h] * 0.5, float(sink[h])) @ rows[lo:t + 1, :dv]
    R = torch.zeros((ring, dk), dtype=torch.bfloat16, device="cuda")
    Q, out, ws, sk = dev(q.reshape(T, -1)), torch.zeros((T, H * dv), device="cuda"), workspace(dv), dev(sink)
    Rall = dev(rows, torch.bfloat16)
    assert L().yalm_attn_latent_mma_shape(dk, dv, dk) == 1
    at = 0
    for n in [1, 1, 3, 2, 1] * 100:
        n = min(n, T - at)
        if n <= 0:
            break
        for p in range(at, at + n):
            R[p % ring] = Rall[p]
        ok(L().yalm_attn_latent_mma_rows(ptr(out[at:]), H * dv, ptr(Q[at:]), H * dk, ptr(R), dk, ptr(ws), n, H, dk, dv, ring, window, f32(0.5), nsplit, at, None, ptr(sk), None),
           "attn_latent_mma_rows")
        at += n
    close_enough(out.cpu().numpy().reshape(T, H, dv), want, 1e-2)     # the weights are bf16 operands of the second product
    if window > 0:                                                   # the crafted queries make the edge count
        other = np.zeros((T, H, dv))
        for t in range(T):
            lo = max(0, t - size)
            for h in range(H):
                other[t, h] = O.softmax_with_sink(rows[lo:t + 1] @ q[t, h] * 0.5, float(sink[h])) @ rows[lo:t + 1, :dv]
        assert np.abs(other - want).max() > 0.1


# ---- small ops -----------------------------------------------------------------------------------------------------------------
def test_maps_combination():
    rng = np.random.default_rng(7)
    n, H, dv, lam, diff, eps = 5, 3, 40, 0.83, 0.35, 1e-5
    a, g = rng.standard_normal((n, 2, H, dv)), rng.standard_normal((n, H + 2))
    o = a[:, 0] - lam * a[:, 1]
    want = O.rms(o, eps) * (1 - diff) * O.sigmoid(g[:, 1:1 + H])[:, :, None]
    out, gd, ad = torch.zeros((n, H * dv), device="cuda"), dev(g), dev(a.reshape(n, -1))
    ok(L().yalm_diff_combine_rows(ptr(out), H * dv, ptr(ad), 2 * H * dv, vp(gd.data_ptr() + 4), H + 2, n, H, dv, f32(lam), f32(1 - diff), f32(eps), None),
       "diff_combine_rows")
    close_enough(out.cpu().numpy().reshape(n, H, dv), want)


def test_exact_gelu():
    z = np.concatenate([np.linspace(-8, 8, 1001), [0.0, -0.0, 30.0, -30.0]])
    h = dev(np.stack([z, z[::-1]]))
    ok(L().yalm_act_rows(ptr(h), len(z), 2, len(z), 4, None), "act_rows")
    close_enough(h.cpu().numpy(), np.stack([O.gelu_erf(z), O.gelu_erf(z[::-1])]), 1e-6)
    assert np.abs(O.gelu_erf(z) - O.gelu_tanh(z)).max() > 1e-4     # the two forms differ by more than the tolerance


@pytest.mark.parametrize("dt,tt", [(api.F32, torch.float32), (api.BF16, torch.bfloat16)])
@pytest.mark.parametrize("W,sd", [(48, 8), (100, 5), (512, 16)])
def test_token_side_input(W, sd, dt, tt):
    rng = np.random.default_rng(W)
    n, V, layers, layer, eps = 7, 30, 3, 1, 1e-5
    w = {"side.embed": O.bf16_round(rng.standard_normal((V, layers * sd))), "l1.side.gate": O.bf16_round(rng.standard_normal((sd, W)) / math.sqrt(W)),
         "l1.side.proj": O.bf16_round(rng.standard_normal((W, sd))), "l1.side.norm": 0.5 + rng.standard_normal(W)}
    x, toks = rng.standard_normal((n, W)), rng.integers(0, V, n)
    want = x + O.token_side(x, toks, layer, {"token_side": {"dim": sd}}, w, eps)
    xd, tab, tk, wg, wp, nw = dev(x), dev(w["side.embed"], tt), dev(toks, torch.int32), dev(w["l1.side.gate"], tt), dev(w["l1.side.proj"], tt), dev(w["l1.side.norm"])
    ok(L().yalm_token_side_rows(ptr(xd), ptr(tab), layers * sd, layer * sd, ptr(tk), None, ptr(wg), ptr(wp), ptr(nw), dt, n, W, sd, f32(eps), None), "token_side_rows")
    close_enough(xd.cpu().numpy(), want)


@pytest.mark.parametrize("dt,tt", [(api.F32, torch.float32), (api.BF16, torch.bfloat16)])
@pytest.mark.parametrize("n", [1, 5, 40])
def test_token_side_input_in_steps(n, dt, tt):
    """The spread route: gate rows per warp (or finished in place after a product), then the projection with the norm as its tail."""
    rng = np.random.default_rng(n)
    W, sd, V, layers, layer, eps = 96, 16, 30, 2, 1, 1e-5
    w = {"side.embed": O.bf16_round(rng.standard_normal((V, layers * sd))), "l1.side.gate": O.bf16_round(rng.standard_normal((sd, W)) / math.sqrt(W)),
         "l1.side.proj": O.bf16_round(rng.standard_normal((W, sd))), "l1.side.norm": 0.5 + rng.standard_normal(W)}
    x, toks = rng.standard_normal((n, W)), rng.integers(0, V, n)
    e = w["side.embed"][toks][:, layer * sd:(layer + 1) * sd]
    want_h = O.gelu_tanh(x @ w["l1.side.gate"].T) * e
    xd, tab, tk, wg = dev(x), dev(w["side.embed"], tt), dev(toks, torch.int32), dev(w["l1.side.gate"], tt)
    h = torch.zeros((n, sd + 4), device="cuda")
    ok(L().yalm_token_side_gate_rows(ptr(h), sd + 4, ptr(xd), W, ptr(tab), layers * sd, layer * sd, ptr(tk), None, ptr(wg), dt, n, W, sd, None), "token_side_gate_rows")
    close_enough(h.cpu().numpy()[:, :sd], want_h)
    g = dev(x @ w["l1.side.gate"].T)
    ok(L().yalm_token_side_gate_rows(ptr(g), sd, None, 0, ptr(tab), layers * sd, layer * sd, ptr(tk), None, None, dt, n, W, sd, None), "token_side_gate_rows in place")
    close_enough(g.cpu().numpy(), want_h)
    # the projection of one row with the norm + residual tail, the next sublayer's norm riding along, and an activation on the input
    nw, nxt, wp = 0.5 + rng.standard_normal(W), 1 + 0.2 * rng.standard_normal(W), dev(w["l1.side.proj"], tt)
    for act, fn in ((-1, lambda z: z), (4, O.gelu_erf), (3, O.gelu_tanh)):
        res, y, out, cnt = dev(x[0]), torch.zeros(W, device="cuda"), torch.zeros(W, device="cuda"), torch.zeros(64, dtype=torch.int32, device="cuda")
        nwd, nxd, hd = dev(nw), dev(nxt), dev(want_h[0])
        ok(L().yalm_gemv_act_norm_residual_norm(ptr(res), ptr(y), ptr(hd), ptr(wp), ptr(nwd), f32(eps), sd, W, dt, act, ptr(nxd), ptr(out), ptr(cnt), None), "gemv_act_norm_residual_norm")
        want_x = x[0] + O.rms_norm(fn(want_h[0]) @ w["l1.side.proj"].T, nw, eps)
        close_enough(res.cpu().numpy(), want_x)
        close_enough(out.cpu().numpy(), O.rms_norm(want_x, nxt, eps))
        assert int(cnt[0]) == 0


# ---- small models -----------------------------------------------------------------------------------------------------------------
def open_model(folder, dtype=api.F32, chunk=None, context=0):
    old = os.environ.get("YALM_STACK_CHUNK")
    if chunk is not None:
        os.environ["YALM_STACK_CHUNK"] = str(chunk)
    try:
        m = api.Model(folder, context, dtype).cuda(0)
    finally:
        if chunk is not None:
            if old is None:
                del os.environ["YALM_STACK_CHUNK"]
            else:
                os.environ["YALM_STACK_CHUNK"] = old
    return m, api.InferenceState(m)


def close(m, s):
    s.close()
    m.close()


def checkpoint(tmp_path, cfg, seed=0, edit=None, **kw):
    W = O.make_weights(cfg, seed, **kw)
    if edit:
        edit(W)
        W = {k: O.bf16_round(v) for k, v in W.items()}
    folder = str(tmp_path / ("m%d" % seed))
    O.write_checkpoint(folder, cfg, W)
    return folder, W


_oracle_runs = {}


def oracle_forward(cfg, W, toks):
    key = (json.dumps(cfg, sort_keys=True), float(sum(np.abs(v).sum() for v in W.values())), tuple(toks))
    if key not in _oracle_runs:
        _oracle_runs[key] = O.forward(cfg, W, toks)
    return _oracle_runs[key]


def tokens_for(cfg, n, seed=1):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def five_layers(**kw):
    return O.make_config([
        O.latent_mixer(),
        O.diff_mixer(),
        dict(O.latent_mixer(heads=2, dim=24, vdim=8, kv_from=0), mlp=None),
        O.diff_mixer(heads=3, kv_heads=3, dim=24, vdim=16, size=7, keep_first=0, rot_dims=24, scaling=False, diff=0.55),
        O.latent_mixer(heads=5, dim=8, rot_dim=16, vdim=40, kv_rank=24, base=500.0),
    ], **kw)


ONE_LAYER = {
    "latent attention": [O.latent_mixer()],
    "latent attention, one head, no feed-forward": [dict(O.latent_mixer(heads=1), mlp=None)],
    "latent attention, sizes all different, no unrotated part": [O.latent_mixer(heads=3, dim=0, rot_dim=12, vdim=40, kv_rank=72)],
    "differential attention": [O.diff_mixer()],
    "differential attention, one key head, no kept tokens, whole heads rotated without scaling": [O.diff_mixer(heads=3, kv_heads=1, dim=12, vdim=40, size=5, keep_first=0, rot_dims=12, scaling=False)],
    "differential attention, every head its own keys, window longer than the prompt, no feed-forward": [dict(O.diff_mixer(heads=2, kv_heads=2, size=100, keep_first=4), mlp=None)],
    "differential attention, nothing rotated, many kept tokens": [O.diff_mixer(heads=6, kv_heads=3, dim=8, vdim=8, size=3, keep_first=9, rot_dims=0, scaling=False, diff=0.8)],
}


@pytest.mark.parametrize("name", list(ONE_LAYER))
@pytest.mark.parametrize("side", [8, 0, 3])
def test_one_layer_models(tmp_path, name, side):
    cfg = O.make_config(ONE_LAYER[name], side=side)
    folder, W = checkpoint(tmp_path, cfg, seed=3)
    T = 40
    toks = tokens_for(cfg, T)
    want, after = O.forward(cfg, W, toks)
    m, s = open_model(folder)
    buf = np.zeros((1, T, cfg["width"]), np.float32)
    m.stack_tap(buf)
    got = s.forward_rows(toks, 0, range(T))
    m.stack_tap(None)
    close(m, s)
    close_enough(buf, after)
    close_enough(got, want)


def test_every_layer_of_a_mixed_model(tmp_path):
    cfg = five_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=5)
    T = 50
    toks = tokens_for(cfg, T)
    want, after = oracle_forward(cfg, W, toks)
    m, s = open_model(folder)
    buf = np.zeros((5, T, cfg["width"]), np.float32)
    m.stack_tap(buf)
    got = s.forward_rows(toks, 0, range(T))
    m.stack_tap(None)
    close(m, s)
    for i in range(5):
        close_enough(buf[i], after[i])
    close_enough(got, want)


@pytest.mark.parametrize("dtype,tol", [(api.F32, F32_TOL), (api.BF16, 5e-2)])
def test_sizes_that_are_no_vector_multiple(tmp_path, dtype, tol):
    """Nothing here is a multiple of 8 (some not of 4): every op takes its scalar route, rows of caches and weights start at odd offsets."""
    cfg = O.make_config([
        O.latent_mixer(heads=3, dim=10, rot_dim=6, vdim=14, kv_rank=18),
        O.diff_mixer(heads=3, kv_heads=1, dim=10, vdim=6, size=9, keep_first=2, rot_dims=4),
        O.latent_mixer(heads=2, dim=5, rot_dim=6, vdim=7, kv_rank=18, kv_from=0),
        O.diff_mixer(heads=5, kv_heads=5, dim=6, vdim=11, size=4, keep_first=1, rot_dims=6, scaling=False),
    ], width=52, vocab=51, ff=36, side=5)
    folder, W = checkpoint(tmp_path, cfg, seed=12)
    T = 45
    toks = tokens_for(cfg, T)
    want, _ = O.forward(cfg, W, toks)
    m, s = open_model(folder, dtype)
    whole = s.forward_rows(toks, 0, range(T))
    s.end_sequence()
    parts = np.concatenate([s.forward_rows(toks[at:at + n], at, range(n)) for at, n in portions(T, [1, 2, 33, 1, 5])])
    close(m, s)
    close_enough(whole, want, tol)
    close_enough(parts, want, tol)


def test_a_left_out_sink_or_a_shifted_window_would_show(tmp_path):
    """The random weights are such that the mechanisms matter: the oracle with the sink removed, or with the window one token
    off, or one kept token fewer, differs from the library by far more than the tolerance."""
    cfg = O.make_config([O.latent_mixer(), O.diff_mixer(size=6, keep_first=2)])
    folder, W = checkpoint(tmp_path, cfg, seed=6)
    toks = tokens_for(cfg, 30)
    m, s = open_model(folder)
    got = s.forward_rows(toks, 0, range(30))
    close(m, s)
    close_enough(got, O.forward(cfg, W, toks)[0])
    no_sink = dict(W, **{"l0.mix.sink": np.full(3, -80.0)})
    assert np.abs(O.forward(cfg, no_sink, toks)[0] - got).max() > 0.05
    for size, keep in ((5, 2), (7, 2), (6, 1), (6, 3)):
        other = json.loads(json.dumps(cfg))
        other["layers"][1]["mixer"]["mask"] = {"size": size, "keep_first": keep}
        assert np.abs(O.forward(other, W, toks)[0] - got).max() > 0.02, (size, keep)


@pytest.mark.parametrize("sizes", [[1], [2], [3, 2, 11, 2, 5], [17, 64]])
def test_whole_prompt_equals_decoding_equals_portions(tmp_path, sizes):
    cfg = five_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=7)
    T = 90
    toks = tokens_for(cfg, T)
    want, _ = oracle_forward(cfg, W, toks)
    m, s = open_model(folder)
    whole = s.forward_rows(toks, 0, range(T))
    s.end_sequence()
    parts = np.concatenate([s.forward_rows(toks[at:at + n], at, range(n)) for at, n in portions(T, sizes)])
    close(m, s)
    close_enough(whole, want)
    close_enough(parts, want)
    close_enough(parts, whole.astype(np.float64))


def test_caches_given_back_and_used_again(tmp_path):
    cfg = five_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=8)
    a, b = tokens_for(cfg, 70, 2), tokens_for(cfg, 33, 3)
    m, s = open_model(folder, chunk=16)
    s.forward_rows(a, 0, [])
    s.end_sequence()
    second = s.forward_rows(b, 0, range(len(b)))
    s.end_sequence()
    m2, s2 = open_model(folder, chunk=16)
    alone = s2.forward_rows(b, 0, range(len(b)))
    close(m2, s2)
    close(m, s)
    np.testing.assert_array_equal(second, alone)                 # nothing of the earlier sequence is read
    close_enough(second, oracle_forward(cfg, W, b)[0])


@pytest.mark.parametrize("chunk", [1, 4, 16])
def test_long_decoding_over_a_wrapping_ring(tmp_path, chunk):
    cfg = five_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=9)
    T = 230
    toks = tokens_for(cfg, T)
    want, _ = oracle_forward(cfg, W, toks)
    m, s = open_model(folder, chunk=chunk)
    assert m.ring_slots(1) == 64 and m.ring_slots(1) < T        # the windowed layer's ring wraps; the kept first tokens live beside it
    rows = sorted(set(list(range(0, T, 7)) + [T - 1]))
    close_enough(s.forward_rows(toks, 0, rows), want[rows])
    s.end_sequence()
    s.forward_rows(toks[:20], 0, [])
    dec = np.concatenate([s.forward_rows(toks[i:i + 1], i, [0]) for i in range(20, T)])
    close(m, s)
    close_enough(dec, want[20:])


def test_prompt_portions_on_the_tensor_cores_and_serving_precision(tmp_path):
    """Head sizes and portions that take the tensor-core products and attention kernels; bf16 against the float64 run, and
    whole = decoded in bf16."""
    cfg = O.make_config([
        O.latent_mixer(heads=4, dim=48, rot_dim=16, vdim=32, kv_rank=64),
        O.diff_mixer(heads=4, kv_heads=2, dim=64, vdim=64, size=50, keep_first=3, rot_dims=32),
        O.latent_mixer(heads=2, dim=112, rot_dim=16, vdim=64, kv_rank=64, kv_from=0),
    ], width=128, vocab=160, ff=256, side=16)
    folder, W = checkpoint(tmp_path, cfg, seed=10)
    T = 150
    toks = tokens_for(cfg, T)
    want, _ = O.forward(cfg, W, toks)
    m, s = open_model(folder, api.F32)
    close_enough(s.forward_rows(toks, 0, range(T)), want)
    close(m, s)
    m, s = open_model(folder, api.BF16)
    whole = s.forward_rows(toks, 0, range(T))
    s.end_sequence()
    cut = np.concatenate([s.forward_rows(toks[at:at + n], at, range(n)) for at, n in portions(T, [70, 33, 47])])
    s.end_sequence()
    s.forward_rows(toks[:100], 0, [])
    dec = np.concatenate([s.forward_rows(toks[i:i + 1], i, [0]) for i in range(100, T)])
    close(m, s)

    def rows_close(got, ref):
        e = np.abs(got - ref).max(1) / max(1.0, np.abs(ref).max())
        assert np.median(e) < 2e-2 and e.max() < 6e-2, (float(np.median(e)), float(e.max()))
    rows_close(whole, want)
    rows_close(cut, want)
    rows_close(dec, want[100:])


def test_generation_through_the_entry_points(tmp_path):
    cfg = five_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=11)
    prompt, n = tokens_for(cfg, 21), 14
    want = O.greedy(cfg, W, prompt, n)
    m, s = open_model(folder)
    assert s.generate(prompt, n) == want
    s.end_sequence()
    s.forward_batch(prompt[:-1], 0)
    assert s.generate_greedy(prompt[-1], len(prompt) - 1, n) == want      # the captured decode step, replayed
    s.end_sequence()
    s.forward_batch(prompt[:-1], 0)
    toks, lg = s.generate_greedy(prompt[-1], len(prompt) - 1, n, keep_logits=True)
    assert toks == want
    close_enough(lg, O.forward(cfg, W, prompt + want)[0][len(prompt) - 1:-1])
    s.end_sequence()
    s.forward_batch(prompt[:-1], 0)
    a = s.generate_sampled(prompt[-1], len(prompt) - 1, n, 0.8, seed=5)
    s.end_sequence()
    s.forward_batch(prompt[:-1], 0)
    b = s.generate_sampled(prompt[-1], len(prompt) - 1, n, 0.8, seed=5)
    close(m, s)
    assert a == b and all(0 <= t < cfg["vocab"] for t in a)


def test_command_line_on_a_checkpoint_directory(tmp_path):
    exe = os.path.join(ROOT, "build", "main")
    if not os.path.exists(exe):
        subprocess.check_call(["make", "-s", "-C", ROOT, "cli"])
    cfg = five_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=15)
    prompt = tokens_for(cfg, 17)
    text = " ".join(map(str, prompt))
    r = subprocess.run([exe, folder, "-m", "completion", "-i", text, "-n", "6", "-t", "0", "-p", "fp32"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    ids = [l for l in r.stdout.splitlines() if re.fullmatch(r"(\d+ )+", l)]
    assert ids and [int(x) for x in ids[-1].split()] == O.greedy(cfg, W, prompt, 6)


def test_trace_runner(tmp_path):
    cfg = five_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=14)
    a, b = tokens_for(cfg, 25, 4), tokens_for(cfg, 9, 5)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": [19, 3, 19]}], "end": []},   # rows come in the order asked
             {"step": 1, "entries": [{"id": "a", "tokens": a[20:22], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[22:], "want": [2]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b, "want": [8]}], "end": ["b"]}]
    out = tmp_path / "out"
    out.mkdir()
    env = dict(os.environ, YALM_B200_LIB=api.LIB_PATH)
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", 5e-2)):
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, env=env, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == ["done 0", "done 1", "done 2", "done 3"]
        wa, wb = O.forward(cfg, W, a)[0], O.forward(cfg, W, b)[0]
        V = cfg["vocab"]
        close_enough(np.fromfile(out / "0.f32", "<f4").reshape(-1, V), wa[[19, 3, 19]], tol)
        assert not (out / "1.f32").exists()
        close_enough(np.fromfile(out / "2.f32", "<f4").reshape(-1, V), wa[[24]], tol)
        close_enough(np.fromfile(out / "3.f32", "<f4").reshape(-1, V), wb[[8]], tol)
        for f in out.iterdir():
            f.unlink()
