"""-m gpu: the Fegizen design on the layered executor against the plain float64 statement in fegizen_oracle.py.

The new row ops alone (device arrays through the C ABI): norm + input convolution in portions shorter than its tail, the
rotary table and both rotations, the windowed attention over rows that hold keys and values together with crafted queries
that single out one key at every edge of the window, the matrix-state recurrence in its gated-linear-attention form with a
key hundreds of positions back, the router with its choice bias, the weighted sum over depth.  Then small models with random
weights whose sizes differ from layer to layer and avoid the equalities a single configuration would hide: every mechanism
through the residual after its layer; whole prompts against token-by-token decoding and portions down to two tokens; state
given back and used again; long decoding over a wrapping ring; serving precision; greedy generation through the library's
entry points, the command line and the trace runner.
"""
import ctypes as C
import json
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

import fegizen_oracle as O
from yalm_b200 import api

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32_TOL = 3e-4
vp, i32, f32, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.ascontiguousarray(a), dtype=dtype).cuda().contiguous()


def ptr(t):
    return vp(t.data_ptr()) if t is not None else None


_alive = []


def devp(a):
    """Pointer to a device copy that stays allocated (a temporary would be freed, and its memory reused, before the launch)."""
    _alive.append(dev(a))
    del _alive[:-64]
    return ptr(_alive[-1])


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


# ---- norm + input convolution -----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("taps", [1, 2, 3, 5])
@pytest.mark.parametrize("sizes", [[1000], [1], [2], [1, 2, 40, 3]])
@pytest.mark.parametrize("layer_norm", [1, 0])
def test_norm_and_input_convolution_in_portions(taps, sizes, layer_norm):
    L = api.lib()
    L.yalm_norm_conv_rows.argtypes = [vp, vp, vp, vp, i32, f32, vp, vp, i32, i32, i32, i32, vp, vp]
    rng = np.random.default_rng(taps)
    T, W, eps = 61, 70, 1e-5
    x = rng.standard_normal((T, W)) * 3 + 1.0
    w, cw = 1 + 0.3 * rng.standard_normal(W), rng.standard_normal((W, taps))
    h = O.layer_norm(x, w, eps) if layer_norm else O.rms_norm(x, w, eps)
    want = O.with_conv(h, cw)
    xd, wd, cd = dev(x), dev(w), dev(cw)
    u, hd = torch.zeros(T, W, device="cuda"), torch.zeros(T, W, device="cuda")
    state = torch.full((max(1, taps - 1), W), 9.0, device="cuda")           # garbage: a call at position 0 must not read it
    for at, n in portions(T, sizes):
        ok(L.yalm_norm_conv_rows(ptr(u[at:]), ptr(hd[at:]), ptr(xd[at:]), ptr(wd), layer_norm, eps, ptr(cd), ptr(state), n, W, taps, at, None, None), "norm_conv_rows")
    close_enough(u.cpu().numpy(), want, 1e-5)
    close_enough(hd.cpu().numpy(), h, 1e-5)
    if taps > 1:
        close_enough(state.cpu().numpy(), h[T - (taps - 1):], 1e-5)


# ---- rotary positions ----------------------------------------------------------------------------------------------------------
def test_rotary_table_by_hand():
    """dims 8, base 10000, factor 4, original 32, fast 4, slow 1: d(t) = 8 ln(32 / (2 pi t)) / (2 ln 10000); d(4) = 0.105 -> lo 0,
    d(1) = 0.707 -> hi 1: pair 0 keeps its frequency, pairs 1 .. 3 are divided by 4; cos and sin times 0.1 ln 4 + 1."""
    f, mag = O.rotary_table({"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "original": 32, "fast": 4.0, "slow": 1.0}})
    np.testing.assert_allclose(f, [1.0, 0.1 / 4, 0.01 / 4, 0.001 / 4], rtol=1e-12)
    assert abs(mag - (0.1 * np.log(4.0) + 1)) < 1e-12


@pytest.mark.parametrize("scaling", [True, False])
@pytest.mark.parametrize("sizes", [[1000], [1], [3, 2]])
def test_latent_rows_norms_rotation_and_cache(scaling, sizes):
    """The packed projection's pieces: query latent normed in place, key / value latent normed and the rotated key part in the
    ring row of their position; then the query map: unrotated part through W_uk, rotated part turned."""
    L = api.lib()
    L.yalm_latent_post_rows.argtypes = [vp, i32, i32, i32, vp, i32, i32, i32, vp, vp, i32, vp, f32, i32, i32, f32, i32, i32, i32, vp, vp]
    L.yalm_latent_query_rows.argtypes = [vp, i32, vp, i32, vp, i32, i32, i32, i32, i32, i32, vp, f32, i32, i32, i32, vp, vp]
    rng = np.random.default_rng(5)
    T, qr, r, dr, H, dn, eps = 37, 20, 12, 6, 3, 10, 1e-5
    ring = 16 if max(sizes) < 16 else 48                                     # a call never holds more rows than the ring has slots
    rot = {"dims": dr, "base": 300.0}
    if scaling:
        rot["scaling"] = {"factor": 8.0, "original": 16, "fast": 6.0, "slow": 1.0}
    freqs, mag = O.rotary_table(rot)
    ld, o_q, o_kv = 3 + qr + r + dr + 2, 3, 3 + qr
    P = rng.standard_normal((T, ld))
    qw, kw = 1 + 0.2 * rng.standard_normal(qr), 1 + 0.2 * rng.standard_normal(r)
    Pd, fd = dev(P), dev(freqs)
    ringbuf = torch.zeros(ring, r + dr, device="cuda")
    q = rng.standard_normal((T, H, dn + dr))
    uk = rng.standard_normal((H * dn, r))
    qd, ukd = dev(q.reshape(T, -1)), dev(uk.reshape(H, dn, r).transpose(0, 2, 1))     # the library takes every head's matrix transposed
    qa = torch.zeros(T, H * (r + dr), device="cuda")
    for at, n in portions(T, sizes):
        ok(L.yalm_latent_post_rows(ptr(Pd[at:]), ld, o_q, qr, devp((qw)), o_kv, r, dr, devp((kw)), ptr(ringbuf), ring, ptr(fd), mag, dr, 1, eps, 1, n, at, None,
                                   None), "latent_post_rows")
        ok(L.yalm_latent_query_rows(ptr(qa[at:]), H * (r + dr), ptr(qd[at:]), H * (dn + dr), ptr(ukd), api.F32, n, H, dn, dr, r, ptr(fd), mag, dr, 1, at, None, None),
           "latent_query_rows")
    got = Pd.cpu().numpy()
    close_enough(got[:, o_q:o_q + qr], O.rms_norm(P[:, o_q:o_q + qr], qw, eps), 1e-5)
    np.testing.assert_array_equal(got[:, :o_q], P[:, :o_q].astype(np.float32))
    c = O.rms_norm(P[:, o_kv:o_kv + r], kw, eps)
    kr = np.stack([O.rotate_pairs(P[t, o_kv + r:o_kv + r + dr], t, freqs, mag) for t in range(T)])
    rows = ringbuf.cpu().numpy()
    for t in range(max(0, T - ring), T):                                             # the last `ring` positions, at slot position % ring
        close_enough(rows[t % ring], np.concatenate([c[t], kr[t]]), 1e-5)
    want = np.zeros((T, H, r + dr))
    for t in range(T):
        for h in range(H):
            want[t, h, :r] = uk[h * dn:(h + 1) * dn].T @ q[t, h, :dn]
            want[t, h, r:] = O.rotate_pairs(q[t, h, dn:], t, freqs, mag)
    close_enough(qa.cpu().numpy().reshape(T, H, -1), want, 1e-5)


def test_rotation_at_large_positions():
    """Angles are position times frequency in fp32: at positions of a few thousand the result still follows the exact rotation."""
    L = api.lib()
    L.yalm_latent_query_rows.argtypes = [vp, i32, vp, i32, vp, i32, i32, i32, i32, i32, i32, vp, f32, i32, i32, i32, vp, vp]
    rng = np.random.default_rng(6)
    dr, r, dn = 8, 4, 4
    freqs, mag = O.rotary_table({"dims": dr, "base": 10000.0})
    q, uk = rng.standard_normal((1, dn + dr)), rng.standard_normal((dn, r))
    out = torch.zeros(1, r + dr, device="cuda")
    for pos in (0, 1, 4095, 100000):
        ok(L.yalm_latent_query_rows(ptr(out), r + dr, devp((q)), dn + dr, devp((uk.T)), api.F32, 1, 1, dn, dr, r, devp((freqs)), mag, dr, 1, pos, None, None), "q rows")
        want = O.rotate_pairs(q[0, dn:], pos, freqs.astype(np.float32).astype(np.float64), mag)
        close_enough(out.cpu().numpy()[0, r:], want, 1e-5 + 2e-7 * pos)


# ---- windowed attention over rows that hold keys and values together -----------------------------------------------------------
def attend(q, rows, dv, window, scale):
    """q (T, H, dk), rows (T, dk): key = the row, value = its first dv channels; position i sees 0 <= i - j < window."""
    T, H, dk = q.shape
    out = np.zeros((T, H, dv))
    for i in range(T):
        lo = max(0, i - window + 1) if window else 0
        for h in range(H):
            s = rows[lo:i + 1] @ q[i, h] * scale
            e = np.exp(s - s.max())
            out[i, h] = (e / e.sum()) @ rows[lo:i + 1, :dv]
    return out


def run_attention(q, rows, dv, window, scale, ring, sizes, cache_f32=1):
    L = api.lib()
    L.yalm_attn_window_pool_strided.argtypes = [vp, i32, vp, i32, vp, i32, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, f32, i32, i32, i32, vp, vp]
    L.yalm_attn_window_pool_workspace.restype = sz
    L.yalm_attn_window_pool_workspace.argtypes = [i32]
    T, H, dk = q.shape
    ws = torch.zeros(L.yalm_attn_window_pool_workspace(dv), device="cuda")
    qd = dev(q.reshape(T, -1))
    ringbuf = torch.full((ring, dk), 50.0, device="cuda", dtype=torch.float32 if cache_f32 else torch.bfloat16)
    rd = dev(rows, torch.float32 if cache_f32 else torch.bfloat16)
    out = torch.zeros(T, H * dv, device="cuda")
    for at, n in portions(T, sizes):
        for t in range(at, at + n):
            ringbuf[t % ring] = rd[t]                                        # what the append leaves: slot = position % ring
        ok(L.yalm_attn_window_pool_strided(ptr(out[at:]), H * dv, ptr(qd[at:]), H * dk, ptr(ringbuf), dk, ptr(ringbuf), dk, None, None, ptr(ws), n, H, 1, dk, dv, ring,
                                           0, window, 0, scale, cache_f32, 4096, at, None, None), "attn_window_pool_strided")
    return out.cpu().numpy().reshape(T, H, dv)


@pytest.mark.parametrize("dk,dv,H", [(20, 12, 3), (176, 144, 6), (72, 64, 5), (13, 7, 1)])
@pytest.mark.parametrize("sizes", [[1000], [1], [2], [7, 1, 30]])
def test_attention_edges_of_the_window(dk, dv, H, sizes):
    """Query i points at one key: the oldest inside the window, the newest outside, position 0, itself.  A window one key
    longer or shorter changes what the pointed queries return, so an edge that is off by one shows."""
    rng = np.random.default_rng(dk)
    T, window = 90, 17
    rows = rng.standard_normal((T, dk))
    rows /= np.linalg.norm(rows, axis=-1, keepdims=True)
    q = rng.standard_normal((T, H, dk)) * 0.1
    target = {}
    for i in range(T):
        j = [i - window + 1, i - window, 0, i][i % 4]
        if 0 <= j <= i:
            q[i, i % H] = 40.0 * rows[j]                                     # score 40 on that key, about 40 cos(angle) elsewhere
            target[i] = j
    want = attend(q, rows, dv, window, 1.0)
    ring = window + max(min(s, T) for s in sizes)
    got = run_attention(q, rows, dv, window, 1.0, ring, sizes)
    close_enough(got, want, 2e-5)
    for other in (window - 1, window + 1):
        assert np.abs(attend(q, rows, dv, other, 1.0) - want).max() > 0.05
    inside = [i for i, j in target.items() if i - j == window - 1 and i % 4 == 0]
    outside = [i for i, j in target.items() if i - j == window]
    assert inside and outside
    for i in inside:
        np.testing.assert_allclose(got[i, i % H], rows[target[i], :dv], atol=2e-3)
    for i in outside:
        assert np.abs(got[i, i % H] - rows[target[i], :dv]).max() > 0.05


def run_attention_one_pass(q, rows, dv, window, scale, ring, sizes):
    """The kernel that reads every bf16 row once for scores and sums."""
    L = api.lib()
    L.yalm_attn_latent_rows.argtypes = [vp, i32, vp, i32, vp, i32, vp, i32, i32, i32, i32, i32, i32, f32, i32, i32, vp, vp]
    L.yalm_attn_window_pool_workspace.restype = sz
    L.yalm_attn_window_pool_workspace.argtypes = [i32]
    T, H, dk = q.shape
    ws = torch.zeros(L.yalm_attn_window_pool_workspace(dv), device="cuda")
    qd = dev(q.reshape(T, -1))
    ringbuf = torch.full((ring, dk), 50.0, device="cuda", dtype=torch.bfloat16)
    rd = dev(rows, torch.bfloat16)
    out = torch.zeros(T, H * dv, device="cuda")
    for at, n in portions(T, sizes):
        for t in range(at, at + n):
            ringbuf[t % ring] = rd[t]
        ok(L.yalm_attn_latent_rows(ptr(out[at:]), H * dv, ptr(qd[at:]), H * dk, ptr(ringbuf), dk, ptr(ws), n, H, dk, dv, ring, window, scale, 4096, at, None, None),
           "attn_latent_rows")
    return out.cpu().numpy().reshape(T, H, dv)


@pytest.mark.parametrize("dk,dv,H", [(24, 16, 3), (176, 144, 6), (320, 256, 2), (576, 512, 5), (72, 57, 1)])
@pytest.mark.parametrize("sizes", [[1000], [1], [2, 1, 30]])
def test_one_pass_attention_edges_of_the_window(dk, dv, H, sizes):
    """The same crafted queries through the kernel that serves bf16 caches; rows are bf16 values, so the comparison is exact
    up to fp32 summation order."""
    rng = np.random.default_rng(dk)
    T, window = 90, 17
    rows = rng.standard_normal((T, dk))
    rows = O.bf16_round(rows / np.linalg.norm(rows, axis=-1, keepdims=True)).astype(np.float64)
    q = rng.standard_normal((T, H, dk)) * 0.1
    target = {}
    for i in range(T):
        j = [i - window + 1, i - window, 0, i][i % 4]
        if 0 <= j <= i:
            q[i, i % H] = 40.0 * rows[j]
            target[i] = j
    want = attend(q, rows, dv, window, 1.0)
    got = run_attention_one_pass(q, rows, dv, window, 1.0, window + max(min(s, T) for s in sizes), sizes)
    close_enough(got, want, 2e-5)
    for other in (window - 1, window + 1):
        assert np.abs(attend(q, rows, dv, other, 1.0) - want).max() > 0.05
    for i, j in target.items():
        if i - j == window - 1 and i % 4 == 0:
            np.testing.assert_allclose(got[i, i % H], rows[j, :dv], atol=3e-3)
        if i - j == window:
            assert np.abs(got[i, i % H] - rows[j, :dv]).max() > 0.05


def test_attention_far_key_without_a_window_and_bf16_rows():
    rng = np.random.default_rng(2)
    T, H, dk, dv = 700, 4, 40, 32
    rows = rng.standard_normal((T, dk))
    rows /= np.linalg.norm(rows, axis=-1, keepdims=True)
    rows = O.bf16_round(rows).astype(np.float64)
    q = rng.standard_normal((T, H, dk)) * 0.1
    q[T - 1, 1] = 60.0 * rows[3]
    want = attend(q, rows, dv, 0, 1.0)
    for f32c in (1, 0):
        got = run_attention(q, rows, dv, 0, 1.0, T, [650, 1], cache_f32=f32c)
        close_enough(got, want, 2e-5)
        np.testing.assert_allclose(got[T - 1, 1], rows[3, :dv], atol=2e-3)
    got = run_attention_one_pass(q, rows, dv, 0, 1.0, T, [650, 1])
    close_enough(got, want, 2e-5)
    np.testing.assert_allclose(got[T - 1, 1], rows[3, :dv], atol=2e-3)


# ---- gated linear attention: the recurrence -----------------------------------------------------------------------------------------
def run_gla(q, k, v, alpha, sizes):
    L = api.lib()
    L.yalm_state_scan_rows.argtypes = [vp, i32, vp, i32, vp, i32, vp, i32, vp, i32, i32, vp, i32, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp]
    T, H, D = q.shape
    P = v.shape[2]
    state = torch.full((H, P, D), 7.0, device="cuda")
    out = torch.zeros(T, H * P, device="cuda")
    kd, qd, vd, ad = dev(k.reshape(T, -1)), dev(q.reshape(T, -1)), dev(v.reshape(T, -1)), dev(alpha.reshape(T, -1))
    for at, n in portions(T, sizes):
        ok(L.yalm_state_scan_rows(ptr(out[at:]), H * P, ptr(kd[at:]), H * D, ptr(qd[at:]), H * D, ptr(vd[at:]), H * P, ptr(ad[at:]), H * D, 1, None, 0, None, 0, None,
                                  ptr(state), n, H, 1, D, P, at, None, None), "state_scan_rows")
    return out.cpu().numpy().reshape(T, H, P)


@pytest.mark.parametrize("D,P,H", [(16, 24, 2), (32, 72, 5), (20, 9, 3), (128, 40, 1)])
@pytest.mark.parametrize("sizes", [[1000], [1], [2, 1, 9, 30]])
def test_gated_linear_attention_recurrence(D, P, H, sizes):
    L = api.lib()
    L.yalm_gla_prep_rows.argtypes = [vp, i32, vp, f32, vp, i32, f32, i32, i32, vp]
    rng = np.random.default_rng(D + P)
    T, tau = 50, 6.0
    q, k, v = rng.standard_normal((T, H, D)), rng.standard_normal((T, H, D)) / np.sqrt(D), rng.standard_normal((T, H, P))
    z, b = 3 * rng.standard_normal((T, H * D)), rng.standard_normal(H * D)
    z[0, 0], z[1, 1] = 40.0, -40.0                                          # saturated either way
    alpha = (1.0 / (1.0 + np.exp(-(z + b)))) ** (1.0 / tau)
    zd, qd = dev(z), dev(q.reshape(T, -1))
    ok(L.yalm_gla_prep_rows(ptr(zd), H * D, devp((b)), tau, ptr(qd), H * D, D ** -0.5, T, H * D, None), "gla_prep_rows")
    close_enough(zd.cpu().numpy(), alpha, 1e-6)
    close_enough(qd.cpu().numpy(), q.reshape(T, -1) * D ** -0.5, 1e-6)
    want = O.gla_scan(q * D ** -0.5, k, v, alpha.reshape(T, H, D))
    got = run_gla(qd.cpu().numpy().reshape(T, H, D).astype(np.float64), k, v, zd.cpu().numpy().reshape(T, H, D).astype(np.float64), sizes)
    close_enough(got, want, 2e-5)


def test_gated_linear_attention_keeps_a_far_key():
    """One key channel never decays and carries a value written 600 positions back; the last query reads exactly that channel."""
    rng = np.random.default_rng(4)
    T, H, D, P = 640, 2, 16, 8
    q, k, v = 0.05 * rng.standard_normal((T, H, D)), 0.05 * rng.standard_normal((T, H, D)), rng.standard_normal((T, H, P))
    alpha = rng.uniform(0.6, 0.9, (T, H, D))
    alpha[:, 1, 5] = 1.0
    k[:, 1, 5] = 0.0
    k[30, 1, 5] = 1.0
    q[T - 1, 1] = 0.0
    q[T - 1, 1, 5] = 1.0
    want = O.gla_scan(q, k, v, alpha)
    np.testing.assert_allclose(want[T - 1, 1], v[30, 1], atol=1e-9)
    for sizes in ([1000], [600, 1], [33]):
        got = run_gla(q, k, v, alpha, sizes)
        close_enough(got, want, 2e-5)
        np.testing.assert_allclose(got[T - 1, 1], v[30, 1], atol=1e-5)


# ---- router, weighted sum over depth ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("E,ident,top", [(5, 2, 2), (11, 3, 4), (3, 0, 3), (1, 1, 1)])
def test_router_with_choice_bias(E, ident, top):
    L = api.lib()
    L.yalm_router_bias_topk_rows.argtypes = [vp, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32, i32, f32, i32, i32, vp, f32, vp]
    rng = np.random.default_rng(E)
    T, W = 40, 24
    h = rng.standard_normal((T, W))
    w = {"r.router": 2.0 * rng.standard_normal((E + ident, W)) / np.sqrt(W), "r.correction": 0.3 * rng.standard_normal(E + ident)}
    f = {"router": {"experts": E, "identity": ident, "top": top, "scale": 2.5}}
    ids, ws = O.route(h, f, w, "r.")
    gi, gw = torch.zeros(T, top, dtype=torch.int32, device="cuda"), torch.zeros(T, top, device="cuda")
    ok(L.yalm_router_bias_topk_rows(ptr(gi), ptr(gw), devp((h)), W, devp((w["r.router"])), api.F32, T, E + ident, top, W, 0, 1, 1e-20, 1, 1,
                                    devp((w["r.correction"])), 2.5, None), "router_bias_topk_rows")
    np.testing.assert_array_equal(gi.cpu().numpy(), ids)
    close_enough(gw.cpu().numpy(), ws, 1e-5)
    if ident and E > 1:
        plain, _ = O.route(h, f, {"r.router": w["r.router"]}, "r.")
        assert (plain != ids).any()                                          # the bias changes choices in this draw


def test_weighted_sum_over_depth():
    L = api.lib()
    L.yalm_depth_average_rows.argtypes = [vp, vp, sz, vp, i32, i32, i32, vp, vp, vp, i32, i32, vp]
    rng = np.random.default_rng(8)
    n, W, cap, count, top = 5, 12, 9, 4, 3
    hist = rng.standard_normal((count, cap, W))
    x, a, b, y = rng.standard_normal((n, W)), rng.standard_normal((n, W)), rng.standard_normal((n, W)), rng.standard_normal((n * top, W))
    w = rng.standard_normal(count)
    res = x + a + b + y.reshape(n, top, W).sum(1)
    hd, xd = dev(hist), dev(x)
    ok(L.yalm_depth_average_rows(ptr(xd), ptr(hd), cap * W, devp((w)), count, n, W, devp((a)), devp((b)), devp((y)), W, top, None), "depth_average_rows")
    close_enough(hd.cpu().numpy()[count - 1, :n], res, 1e-6)
    close_enough(xd.cpu().numpy(), sum(w[j] * hist[j, :n] for j in range(count - 1)) + w[count - 1] * res, 1e-6)


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
    """O.forward, remembered per (configuration, weights, tokens): parametrised tests share their slow float64 runs."""
    key = (json.dumps(cfg, sort_keys=True), float(sum(np.abs(v).sum() for v in W.values())), tuple(toks))
    if key not in _oracle_runs:
        _oracle_runs[key] = O.forward(cfg, W, toks)
    return _oracle_runs[key]


def tokens_for(cfg, n, seed=1):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def five_layers(**kw):
    return O.make_config([
        ("latent_attention", O.latent_mixer(), O.moe_mlp()),
        ("gla", O.gla_mixer(), O.dense_mlp()),
        ("latent_attention", O.latent_mixer(heads=3, dim=12, vdim=20, window=7, kv_from=0), None),
        ("gla_2", O.gla_mixer(heads=3, dim=20, vdim=8, tau=3.0), O.moe_mlp(ff=16, experts=3, identity=0, top=3, scale=1.0, shared=0)),
        ("latent_attention", O.latent_mixer(heads=5, dim=24, rot_dim=16, vdim=8, kv_rank=40, q_rank=16, window=30), O.dense_mlp(ff=40)),
    ], **kw)


ONE_LAYER = {
    "latent attention": [("latent_attention", O.latent_mixer(), O.dense_mlp())],
    "latent attention, plain frequencies, one head, no feed-forward": [("latent_attention", O.latent_mixer(heads=1, scaling=False, window=5), None)],
    "latent attention, sizes all different": [("latent_attention", O.latent_mixer(heads=3, dim=24, rot_dim=4, vdim=40, kv_rank=72, q_rank=8, window=9), O.dense_mlp(ff=24))],
    "linear attention": [("gla", O.gla_mixer(), O.dense_mlp())],
    "linear attention, wide values, no feed-forward": [("gla_2", O.gla_mixer(heads=3, dim=8, vdim=40, tau=1.0), None)],
    "experts with identity experts and a shared expert": [("gla", O.gla_mixer(), O.moe_mlp())],
    "experts, all chosen, none identity, no shared expert": [("gla", O.gla_mixer(), O.moe_mlp(experts=4, identity=0, top=4, shared=0, scale=1.0))],
    "experts, one real expert among identity experts": [("gla", O.gla_mixer(), O.moe_mlp(experts=1, identity=3, top=2))],
}


@pytest.mark.parametrize("name", list(ONE_LAYER))
@pytest.mark.parametrize("taps", [3, 1, 4])
def test_one_layer_models(tmp_path, name, taps):
    cfg = O.make_config(ONE_LAYER[name], taps=taps)
    folder, W = checkpoint(tmp_path, cfg, seed=3, router_gain=4.0)
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


def test_shared_cache_with_a_wider_window_than_its_owner(tmp_path):
    cfg = O.make_config([("latent_attention", O.latent_mixer(window=4), None), ("latent_attention", O.latent_mixer(window=19, kv_from=0, heads=2), O.dense_mlp())])
    folder, W = checkpoint(tmp_path, cfg, seed=4)
    T = 75
    toks = tokens_for(cfg, T)
    want, _ = O.forward(cfg, W, toks)
    m, s = open_model(folder, chunk=8)
    assert m.ring_slots(0) == 64 and m.ring_slots(1) == 64
    got = s.forward_rows(toks, 0, range(T))
    s.end_sequence()
    s.forward_rows(toks[:3], 0, [])
    dec = np.concatenate([s.forward_rows(toks[i:i + 1], i, [0]) for i in range(3, T)])
    close(m, s)
    close_enough(got, want)
    close_enough(dec, want[3:])


def test_sizes_that_are_no_vector_multiple(tmp_path):
    """Width, vocabulary, latent and head sizes that are not multiples of 4 or 8: every product and row op on its scalar route."""
    cfg = O.make_config([
        ("latent_attention", O.latent_mixer(heads=3, dim=7, rot_dim=6, vdim=5, kv_rank=11, q_rank=9, window=8), O.moe_mlp(ff=10, experts=3, identity=1, top=2, shared=7)),
        ("gla", O.gla_mixer(heads=3, dim=9, vdim=7, tau=2.0), O.dense_mlp(ff=13)),
        ("latent_attention", O.latent_mixer(heads=2, dim=5, rot_dim=6, vdim=9, kv_rank=11, q_rank=6, window=20, kv_from=0), None),
    ], width=50, vocab=70, taps=2)
    folder, W = checkpoint(tmp_path, cfg, seed=21, a_rank=3, router_gain=4.0)
    T = 60
    toks = tokens_for(cfg, T)
    want, after = O.forward(cfg, W, toks)
    for dtype, tol in ((api.F32, F32_TOL), (api.BF16, 6e-2)):
        m, s = open_model(folder, dtype)
        whole = s.forward_rows(toks, 0, range(T))
        s.end_sequence()
        s.forward_rows(toks[:31], 0, [])
        dec = np.concatenate([s.forward_rows(toks[i:i + 1], i, [0]) for i in range(31, T)])
        close(m, s)
        close_enough(whole, want, tol)
        close_enough(dec, want[31:], tol)


def test_keys_and_values_written_out_per_head():
    """The prompt route's helpers: latents of a row range gathered from the ring, then per-head rings of [unrotated key | rotated
    key part] and values; the in-place rotation of the queries and the gate."""
    L = api.lib()
    L.yalm_latent_gather_rows16.argtypes = [vp, vp, i32, i32, i32, i32, i32, vp]
    L.yalm_latent_pack_rings.argtypes = [vp, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp]
    L.yalm_rotate_heads_rows.argtypes = [vp, i32, i32, i32, i32, vp, f32, i32, i32, i32, i32, vp, vp]
    L.yalm_sigmoid_gate_rows.argtypes = [vp, i32, vp, i32, i32, i32, vp]
    rng = np.random.default_rng(9)
    ring, r, dr, H, dn, dv, ring_out = 24, 16, 6, 3, 10, 5, 40
    first, count = 30, 20                                                    # positions 30 .. 49: slots wrap in both rings
    rows = O.bf16_round(rng.standard_normal((ring, r + dr)))
    ringbuf = dev(rows, torch.bfloat16)
    lat = torch.zeros(count, r, device="cuda", dtype=torch.bfloat16)
    ok(L.yalm_latent_gather_rows16(ptr(lat), ptr(ringbuf), ring, r + dr, r, first, count, None), "latent_gather_rows16")
    want_lat = np.stack([rows[(first + j) % ring, :r] for j in range(count)])
    np.testing.assert_array_equal(lat.float().cpu().numpy(), want_lat)
    kv = rng.standard_normal((count, H * (dn + dv)))
    kout = torch.zeros(H, ring_out, dn + dr, device="cuda", dtype=torch.bfloat16)
    vout = torch.zeros(H, ring_out, dv, device="cuda", dtype=torch.bfloat16)
    ok(L.yalm_latent_pack_rings(ptr(kout), ptr(vout), devp((kv)), H * (dn + dv), ptr(ringbuf), ring, r, dr, H, dn, dv, ring_out, first, count, None), "latent_pack_rings")
    kg, vg = kout.float().cpu().numpy(), vout.float().cpu().numpy()
    for j in range(count):
        p = first + j
        for h in range(H):
            np.testing.assert_array_equal(kg[h, p % ring_out, :dn], O.bf16_round(kv[j, h * dn:(h + 1) * dn]))
            np.testing.assert_array_equal(kg[h, p % ring_out, dn:], rows[p % ring, r:])
            np.testing.assert_array_equal(vg[h, p % ring_out], O.bf16_round(kv[j, H * dn + h * dv:H * dn + (h + 1) * dv]))
    freqs, mag = O.rotary_table({"dims": 4, "base": 50.0, "scaling": {"factor": 2.0, "original": 8, "fast": 4.0, "slow": 1.0}})
    n, hs = 7, dn + dr
    q = rng.standard_normal((n, H, hs))
    qd = dev(q.reshape(n, -1))
    ok(L.yalm_rotate_heads_rows(ptr(qd), H * hs, H, hs, dn, devp((freqs)), mag, 4, 1, n, 100, None, None), "rotate_heads_rows")
    want = q.copy()
    for t in range(n):
        for h in range(H):
            want[t, h, dn:] = O.rotate_pairs(q[t, h, dn:], 100 + t, freqs, mag)      # 4 of the 6 channels turn, 2 pass unchanged
    close_enough(qd.cpu().numpy().reshape(n, H, hs), want, 1e-5)
    x, g = rng.standard_normal((n, 11)), rng.standard_normal((n, 13))
    xd = dev(x)
    ok(L.yalm_sigmoid_gate_rows(ptr(xd), 11, devp((g)), 13, n, 9, None), "sigmoid_gate_rows")
    want = x.copy()
    want[:, :9] /= 1 + np.exp(-g[:, :9])
    close_enough(xd.cpu().numpy(), want, 1e-6)


def test_whole_prompt_decoding_and_portions_agree(tmp_path):
    cfg = five_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=5, router_gain=4.0)
    T = 90
    toks = tokens_for(cfg, T)
    want, after = O.forward(cfg, W, toks)
    m, s = open_model(folder)
    buf = np.zeros((5, T, cfg["width"]), np.float32)
    m.stack_tap(buf)
    whole = s.forward_rows(toks, 0, range(T))
    m.stack_tap(None)
    close_enough(buf, after)
    close_enough(whole, want)
    s.end_sequence()
    one = np.concatenate([s.forward_rows(toks[i:i + 1], i, [0]) for i in range(T)])     # from the first token on
    close_enough(one, want)
    s.end_sequence()
    cuts, at, got = [2, 3, 17, 1, 2, 29, 2, 5, 1, 1, 2, 25], 0, []
    assert sum(cuts) == T
    for n in cuts:
        rows = [r for r in range(n) if (at + r) % 3 != 1]
        got.append((np.array(rows) + at, s.forward_rows(toks[at:at + n], at, rows)))
        at += n
    for rows, lg in got:
        if len(rows):
            close_enough(lg, want[rows])
    close(m, s)


def test_state_given_back_and_used_again(tmp_path):
    cfg = five_layers(taps=2)
    folder, W = checkpoint(tmp_path, cfg, seed=8, router_gain=4.0)
    a, b = tokens_for(cfg, 70, 2), tokens_for(cfg, 33, 3)
    m, s = open_model(folder, chunk=8)
    s.forward_rows(a, 0, [])
    s.end_sequence()
    second = s.forward_rows(b, 0, range(len(b)))
    close_enough(second, O.forward(cfg, W, b)[0])
    s.forward_rows(a[:10], 0, [])                     # abandoned: the next sequence starts over at position 0
    with pytest.raises(api.YalmError):
        s.forward_rows(a[10:12], 15, [])
    third = s.forward_rows(b, 0, range(len(b)))
    close(m, s)
    np.testing.assert_array_equal(second, third)


@pytest.mark.parametrize("chunk", [1, 4, 16])
def test_long_decoding_over_a_wrapping_ring(tmp_path, chunk):
    cfg = five_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=9, router_gain=4.0)
    T = 230
    toks = tokens_for(cfg, T)
    want, _ = oracle_forward(cfg, W, toks)
    m, s = open_model(folder, chunk=chunk)
    assert m.ring_slots(0) == 64 and m.ring_slots(0) < T
    rows = sorted(set(list(range(0, T, 7)) + [T - 1]))
    close_enough(s.forward_rows(toks, 0, rows), want[rows])
    s.end_sequence()
    s.forward_rows(toks[:20], 0, [])
    dec = np.concatenate([s.forward_rows(toks[i:i + 1], i, [0]) for i in range(20, T)])
    close(m, s)
    close_enough(dec, want[20:])


def test_prompt_portions_on_the_tensor_cores_and_serving_precision(tmp_path):
    """Widths and portions large enough for the tensor-core products and the grouped experts; bf16 against the float64 run by
    row-wise quantiles (a rounded router input may flip a close choice), and whole = decoded in bf16."""
    cfg = O.make_config([
        ("latent_attention", O.latent_mixer(heads=4, dim=48, rot_dim=16, vdim=32, kv_rank=64, q_rank=48, window=50), O.moe_mlp(ff=64, experts=6, identity=2, top=2, shared=32)),
        ("gla", O.gla_mixer(heads=2, dim=32, vdim=64), O.dense_mlp(ff=128)),
        ("latent_attention", O.latent_mixer(heads=2, dim=112, rot_dim=16, vdim=64, kv_rank=64, q_rank=48, window=20, kv_from=0), O.moe_mlp(ff=64, experts=6, identity=2, top=2, shared=32)),
    ], width=128, vocab=160)
    folder, W = checkpoint(tmp_path, cfg, seed=10, a_rank=8, router_gain=6.0)
    T = 150
    toks = tokens_for(cfg, T)
    want, _ = O.forward(cfg, W, toks)
    m, s = open_model(folder, api.F32)
    close_enough(s.forward_rows(toks, 0, range(T)), want)
    close(m, s)
    m, s = open_model(folder, api.BF16)
    whole = s.forward_rows(toks, 0, range(T))
    s.end_sequence()
    s.forward_rows(toks[:100], 0, [])
    dec = np.concatenate([s.forward_rows(toks[i:i + 1], i, [0]) for i in range(100, T)])
    close(m, s)

    def rows_close(got, ref):
        e = np.abs(got - ref).max(1) / max(1.0, np.abs(ref).max())
        assert np.median(e) < 2e-2 and (e > 6e-2).mean() <= 0.1, (float(np.median(e)), float(e.max()))
    rows_close(whole, want)
    rows_close(dec, want[100:])


def test_generation_through_the_entry_points(tmp_path):
    cfg = five_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=11, router_gain=4.0)
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
    folder, W = checkpoint(tmp_path, cfg, seed=15, router_gain=4.0)
    prompt = tokens_for(cfg, 17)
    text = " ".join(map(str, prompt))
    r = subprocess.run([exe, folder, "-m", "completion", "-i", text, "-n", "6", "-t", "0", "-p", "fp32"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    ids = [l for l in r.stdout.splitlines() if re.fullmatch(r"(\d+ )+", l)]
    assert ids and [int(x) for x in ids[-1].split()] == O.greedy(cfg, W, prompt, 6)


def test_trace_runner(tmp_path):
    cfg = five_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=14, router_gain=4.0)
    a, b = tokens_for(cfg, 25, 4), tokens_for(cfg, 9, 5)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": [3, 19]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[20:22], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[22:], "want": [2]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b, "want": [8]}], "end": ["b"]}]
    out = tmp_path / "out"
    out.mkdir()
    env = dict(os.environ, YALM_B200_LIB=api.LIB_PATH)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == ["done 0", "done 1", "done 2", "done 3"]
    wa, wb = O.forward(cfg, W, a)[0], O.forward(cfg, W, b)[0]
    V = cfg["vocab"]
    close_enough(np.fromfile(out / "0.f32", "<f4").reshape(-1, V), wa[[3, 19]])
    assert not (out / "1.f32").exists()
    close_enough(np.fromfile(out / "2.f32", "<f4").reshape(-1, V), wa[[24]])
    close_enough(np.fromfile(out / "3.f32", "<f4").reshape(-1, V), wb[[8]])
