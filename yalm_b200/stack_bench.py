"""`bench.py --workload retezen-sizes`: prefill and decode throughput of the Retezen design at sizes that resemble a real
model's layers (random weights, bf16), beside the library's closest existing model at equal size (the Llama / Mixtral style
block of the `.yalm` models: same width, heads, head size, feed-forward size, experts, layer count, fp16 weights).

Per size and feed-forward kind it reports
  prefill tok/s   a `context`-token prompt through Model::forward_batch (host-timed around the synchronous calls)
  decode tok/s    greedy steps at the end of that context through Model::generate (CUDA events on the launching stream)
and the share of the HBM / tensor rooflines they reach: decode against the bytes one token must read (Config::active_bytes'
arithmetic: the layer's matrices, the window of keys and values, the pooled blocks), prefill against 2 x parameters x
tokens + attention FLOP.  One JSON line with a `sizes` list; the contract keys carry the first size's decode number.
"""
import json
import os
import shutil
import struct
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# name: width, heads, kv_heads, head size, window, pool, feed-forward size, experts, top, layers, vocab
SIZES = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, window=1024, pool=64, ff=8192, moe_ff=2048, experts=8, top=2, layers=4, vocab=32000),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, window=2048, pool=64, ff=14336, moe_ff=3584, experts=8, top=2, layers=3, vocab=32000),
}
CONTEXT = 4096


def _bf16(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def write_retezen(folder, z, kind, context):
    """A checkpoint directory of the given size; matrices are tiled from one random block (values only matter for timing
    through the router's choices, which stay spread because every expert's rows differ by a shift)."""
    os.makedirs(folder, exist_ok=True)
    rng = np.random.default_rng(1)
    block = _bf16(rng.standard_normal(1 << 22).astype(np.float32) * 0.02)
    W, H, G, D = z["width"], z["heads"], z["kv_heads"], z["dim"]
    mlp = {"kind": "dense", "ff": z["ff"], "limit": 7.0} if kind == "dense" else \
        {"kind": "moe", "expert": {"ff": z["moe_ff"]}, "router": {"experts": z["experts"], "top": z["top"]}}
    layer = {"type": "attention", "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "mask": {"size": z["window"], "pool": z["pool"]},
                                            "scale": D ** -0.5, "v_mix": True}, "mlp": mlp}
    cfg = {"architecture": "Retezen", "width": W, "vocab": z["vocab"], "max_positions": context, "norm": {"eps": 1e-5}, "logit_scale": 1.0,
           "layers": [layer] * z["layers"]}
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    shapes = {"embed": (z["vocab"], W), "pos": (context, W), "final.norm": (W,), "head": (z["vocab"], W)}
    for i in range(z["layers"]):
        p = "l%d." % i
        shapes.update({p + "norm1": (W,), p + "norm2": (W,), p + "mix.q": (H * D, W), p + "mix.k": (G * D, W), p + "mix.v": (G * D, W),
                       p + "mix.o": (W, H * D), p + "mix.q.norm": (H * D,), p + "mix.k.norm": (G * D,), p + "mix.vmix": ()})
        if kind == "dense":
            shapes.update({p + "mlp.gate": (z["ff"], W), p + "mlp.up": (z["ff"], W), p + "mlp.down": (W, z["ff"])})
        else:
            shapes[p + "mlp.router"] = (z["experts"], W)
            for e in range(z["experts"]):
                shapes.update({p + "mlp.e%d.gate" % e: (z["moe_ff"], W), p + "mlp.e%d.up" % e: (z["moe_ff"], W), p + "mlp.e%d.down" % e: (W, z["moe_ff"])})
    header, off = {}, 0
    for name, shp in shapes.items():
        n = int(np.prod(shp)) if shp else 1
        header[name] = {"dtype": "BF16", "shape": list(shp), "data_offsets": [off, off + 2 * n]}
        off += 2 * n
    h = json.dumps(header).encode()
    h += b" " * (-len(h) % 8)
    one = _bf16(np.ones(1, np.float32))[0]
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h)
        for k, (name, shp) in enumerate(shapes.items()):
            n = int(np.prod(shp)) if shp else 1
            if name.endswith(".q.norm") or name.endswith(".k.norm"):
                f.write(np.full(n, one, np.uint16).tobytes())
            elif len(shp) < 2:
                f.write(block[:n].tobytes())
            else:
                f.write(np.resize(np.roll(block, 7919 * k), n).tobytes())
    return cfg


def retezen_numbers(z, kind):
    """-> (weight parameters per token in the layers and head, decode bytes per token at CONTEXT, prefill FLOP per token)"""
    W, H, G, D = z["width"], z["heads"], z["kv_heads"], z["dim"]
    attn = (2 * H * D + 2 * G * D) * W
    ffn = 3 * z["ff"] * W if kind == "dense" else z["top"] * 3 * z["moe_ff"] * W + z["experts"] * W
    params = z["layers"] * (attn + ffn) + z["vocab"] * W
    seen = min(CONTEXT, z["window"])
    blocks = max(0, (CONTEXT - z["window"]) // z["pool"])
    kv = z["layers"] * (seen * 2 * G * D * 2 + blocks * 2 * G * D * 4)
    flop = 2.0 * (params - z["vocab"] * W) + 4.0 * z["layers"] * H * D * (seen + blocks)
    return params, 2 * params + kv, flop


# ---- Fapudra ---------------------------------------------------------------------------------------------------------------
# name: width; attention (left) heads / kv heads / head size / window / kept first tokens; delta rule (right) heads x (dim, vdim)
# and low-rank size; state-space heads x vdim, state; experts; layer order (p = parallel mixer, s = state space)
FAPUDRA_SIZES = {
    "w1024": dict(width=1024, heads=8, kv_heads=2, dim=128, window=1024, keep=4, rheads=8, rdim=128, rvdim=128, rank=64, sheads=32, svdim=64, state=128,
                  moe_ff=1024, experts=8, top=2, groups=4, keep_groups=2, order="pssp", vocab=32000),
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, window=1024, keep=4, rheads=16, rdim=128, rvdim=128, rank=64, sheads=64, svdim=64, state=128,
                  moe_ff=2048, experts=8, top=2, groups=4, keep_groups=2, order="pssp", vocab=32000),
}


def write_fapudra(folder, z, context):
    """A checkpoint directory of the given size: matrices tiled from one random block, norm weights 1."""
    os.makedirs(folder, exist_ok=True)
    rng = np.random.default_rng(2)
    block = _bf16(rng.standard_normal(1 << 22).astype(np.float32) * 0.02)
    W, conv = z["width"], 4
    mlp = {"kind": "moe", "expert": {"ff": z["moe_ff"], "limit": 7.0},
           "router": {"experts": z["experts"], "top": z["top"], "groups": {"count": z["groups"], "keep": z["keep_groups"]}}}
    par = {"type": "parallel", "mlp": mlp,
           "mixer": {"left": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "bias_max": 512, "scale": z["dim"] ** -0.5,
                              "mask": {"size": z["window"], "keep_first": z["keep"]}},
                     "right": {"heads": z["rheads"], "kv_heads": z["rheads"], "dim": z["rdim"], "vdim": z["rvdim"], "conv": conv},
                     "left_scale": 1.0, "right_scale": 1.0}}
    ssm = {"type": "mamba2", "mlp": mlp, "mixer": {"heads": z["sheads"], "vdim": z["svdim"], "state": z["state"], "groups": 1, "norm_groups": 1, "conv": conv}}
    layers = [par if c == "p" else ssm for c in z["order"]]
    cfg = {"architecture": "Fapudra", "width": W, "vocab": z["vocab"], "max_positions": context, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
           "logit_softcap": 30.0, "layers": layers}
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    shapes = {"embed": (z["vocab"], W), "pos": (context, W), "embed.norm": (), "final.norm": (), "head": (z["vocab"], W)}
    for i, c in enumerate(z["order"]):
        p = "l%d." % i
        shapes.update({p + "norm1": (), p + "shift": (W,), p + "mlp.router": (z["experts"], W)})
        for e in range(z["experts"]):
            shapes.update({p + "mlp.e%d.gate" % e: (z["moe_ff"], W), p + "mlp.e%d.up" % e: (z["moe_ff"], W), p + "mlp.e%d.down" % e: (W, z["moe_ff"])})
        if c == "p":
            nq, nk = z["heads"] * z["dim"], z["kv_heads"] * z["dim"]
            rk, rv, rg = z["rheads"] * z["rdim"], z["rheads"] * z["rvdim"], z["rheads"] * z["rdim"]
            a, b = p + "mix.left.", p + "mix.right."
            shapes.update({a + "q": (nq, W), a + "q.b": (nq,), a + "k": (nk, W), a + "k.b": (nk,), a + "rel": (32, z["heads"]), a + "pb": (z["heads"],),
                           a + "g": (nq, W), a + "o": (W, nq),
                           b + "q": (rk, W), b + "k": (rk, W), b + "v": (rv, W), b + "q.conv": (rk, conv), b + "k.conv": (rk, conv), b + "v.conv": (rv, conv),
                           b + "b": (z["rheads"], W), b + "A_log": (z["rheads"],), b + "norm": (z["rvdim"],), b + "a1": (z["rank"], W), b + "a2": (rg, z["rank"]),
                           b + "dt_bias": (rg,), b + "g1": (z["rank"], W), b + "g2": (rv, z["rank"]), b + "o": (W, rv)})
        else:
            inner, ch = z["sheads"] * z["svdim"], z["sheads"] * z["svdim"] + 2 * z["state"]
            m = p + "mix."
            shapes.update({m + "in": (2 * inner + 2 * z["state"] + z["sheads"], W), m + "conv": (ch, conv), m + "conv.b": (ch,), m + "dt_bias": (z["sheads"],),
                           m + "A_log": (z["sheads"],), m + "D": (z["sheads"],), m + "norm": (inner,), m + "o": (W, inner)})
    header, off = {}, 0
    for name, shp in shapes.items():
        n = int(np.prod(shp)) if shp else 1
        header[name] = {"dtype": "BF16", "shape": list(shp), "data_offsets": [off, off + 2 * n]}
        off += 2 * n
    h = json.dumps(header).encode()
    h += b" " * (-len(h) % 8)
    one = _bf16(np.ones(1, np.float32))[0]
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h)
        for k, (name, shp) in enumerate(shapes.items()):
            n = int(np.prod(shp)) if shp else 1
            if not shp or name.endswith(".norm"):
                f.write(np.full(n, one, np.uint16).tobytes())
            elif len(shp) < 2:
                f.write(block[:n].tobytes())
            else:
                f.write(np.resize(np.roll(block, 7919 * k), n).tobytes())
    return cfg


def fapudra_numbers(z):
    """-> (decode bytes per token at CONTEXT, prefill FLOP per token): the active matrices once (bf16), the fp32 matrix states read
    and written, the window of keys; 2 FLOP per active parameter plus the attention's and the recurrences' own products."""
    W = z["width"]
    experts = z["top"] * 3 * z["moe_ff"] * W + z["experts"] * W
    params, state, extra = z["vocab"] * W, 0, 0.0
    for c in z["order"]:
        if c == "p":
            nq, nk = z["heads"] * z["dim"], z["kv_heads"] * z["dim"]
            rk, rv = z["rheads"] * z["rdim"], z["rheads"] * z["rvdim"]
            params += (3 * nq + nk) * W + (2 * rk + 2 * rv + z["rheads"] + 2 * z["rank"]) * W + z["rank"] * (rk + rv) + experts
            seen = min(CONTEXT, z["window"]) + z["keep"]
            state += seen * nk * 2 + 2 * 4 * z["rheads"] * z["rdim"] * z["rvdim"]
            extra += 4.0 * nq * seen + 8.0 * z["rheads"] * z["rdim"] * z["rvdim"]
        else:
            inner = z["sheads"] * z["svdim"]
            params += (3 * inner + 2 * z["state"] + z["sheads"]) * W + experts
            state += 2 * 4 * inner * z["state"]
            extra += 6.0 * inner * z["state"]
    return 2 * params + state, 2.0 * (params - z["vocab"] * W) + extra


def run_fapudra(args, base, emit, shm_path, ClockSampler):
    """`bench.py --workload fapudra-sizes`: the Fapudra design beside the closest existing model on the same executor, Retezen
    with routed experts, at equal width, heads, window, experts, layers and vocabulary."""
    import torch
    from yalm_b200 import api
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peaks = json.load(open(pk)) if os.path.exists(pk) else {"hbm_gbs": 6650.0, "bf16_tflops_sustained": 1400.0}
    hbm, tflops = float(peaks["hbm_gbs"]), float(peaks["bf16_tflops_sustained"])
    steps = max(8, min(args.steps, 128))
    clocks = ClockSampler(0)
    clocks.start()
    out, launches = [], 0

    def measure(model, ids):
        st = api.InferenceState(model)
        st.forward_batch(ids[:1024], 0)                     # warm-up (sizes kernels, first-use set-up)
        st.end_sequence()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        st.forward_batch(ids[:-1], 0)
        t_pre = time.perf_counter() - t0
        st.generate_greedy(ids[-1], CONTEXT - 1, max(3, args.warmup))   # first step eager + graph capture, untimed
        st.generate_greedy(ids[0], CONTEXT - 1 + max(3, args.warmup), steps)
        t_dec = st.device_ms / 1e3
        n = model.launches()
        st.close()
        return (CONTEXT - 1) / t_pre, steps / t_dec, n

    for name, z in FAPUDRA_SIZES.items():
        ids = [(i * 7919 + 1) % z["vocab"] for i in range(CONTEXT)]
        row = {"size": name, "width": z["width"], "layers": z["order"], "context": CONTEXT, "window": z["window"]}
        folder = shm_path("yalm_bench_fapudra_%s_%d" % (name, os.getpid()))
        try:
            write_fapudra(folder, z, CONTEXT + steps + args.warmup + 8)
            model = api.Model(folder, 0, api.BF16).cuda(0)
        finally:
            shutil.rmtree(folder, ignore_errors=True)
        pre, dec, n = measure(model, ids)
        model.close()
        dec_bytes, pre_flop = fapudra_numbers(z)
        launches += steps * n
        row["fapudra"] = {"prefill_tok_s": pre, "decode_tok_s": dec, "prefill_frac_of_measured_bf16": pre_flop * pre / 1e12 / tflops,
                          "decode_frac_of_measured_hbm": dec_bytes * dec / 1e9 / hbm, "decode_bytes_per_token": dec_bytes, "launches_per_token": n}
        zr = dict(z, pool=64, ff=0, layers=len(z["order"]))
        folder = shm_path("yalm_bench_retezen_%s_%d" % (name, os.getpid()))
        try:
            write_retezen(folder, zr, "moe", CONTEXT + steps + args.warmup + 8)
            model = api.Model(folder, 0, api.BF16).cuda(0)
        finally:
            shutil.rmtree(folder, ignore_errors=True)
        pre, dec, n = measure(model, ids)
        model.close()
        _, r_bytes, r_flop = retezen_numbers(zr, "moe")
        row["equal_size_retezen"] = {"prefill_tok_s": pre, "decode_tok_s": dec, "prefill_frac_of_measured_bf16": r_flop * pre / 1e12 / tflops,
                                     "decode_frac_of_measured_hbm": r_bytes * dec / 1e9 / hbm, "decode_bytes_per_token": r_bytes, "launches_per_token": n}
        out.append(row)
    clk = clocks.stop()
    first = out[0]["fapudra"]
    emit(dict(base, impl="ours", metric="batch-1 decode tok/s (Fapudra, first size; all sizes under `sizes`)", value=first["decode_tok_s"], steps=steps,
              ms_per_step=1000.0 / first["decode_tok_s"], dtype="bf16", clocks=clk, gpu_launches=launches, sizes=out,
              e2e={"value": first["decode_tok_s"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 4,
                   "note": "device loop: token ids stay on the device, 4 bytes per token come back"},
              config=dict(base["config"], workload="Fapudra at model-like sizes beside the equal-size Retezen stack", context=CONTEXT,
                          l2="inputs larger than L2 (weights streamed per token)")))


# ---- Fegizen ---------------------------------------------------------------------------------------------------------------
# name: width; latent attention heads x (dim unrotated + rot rotated) keys, vdim values, latent sizes, window; linear attention
# heads x (dim, vdim) and the decay's low-rank size; experts (+ identity experts, shared expert); layer order (l = latent
# attention with experts, s = latent attention reading the first layer's cache, g = linear attention)
FEGIZEN_SIZES = {
    "w1024": dict(width=1024, heads=8, dim=64, rot=64, vdim=128, kv_rank=256, q_rank=512, window=1024, gheads=8, gdim=128, gvdim=128, rank=64,
                  moe_ff=1024, experts=8, identity=2, top=2, shared=1024, order="lggs", vocab=32000),
    "w2048": dict(width=2048, heads=16, dim=64, rot=64, vdim=128, kv_rank=512, q_rank=1024, window=1024, gheads=16, gdim=128, gvdim=128, rank=64,
                  moe_ff=2048, experts=8, identity=2, top=2, shared=2048, order="lggs", vocab=32000),
}


def write_fegizen(folder, z):
    """A checkpoint directory of the given size: matrices tiled from one random block, norm weights 1, depth weights 1 on the
    newest result."""
    os.makedirs(folder, exist_ok=True)
    rng = np.random.default_rng(3)
    block = _bf16(rng.standard_normal(1 << 22).astype(np.float32) * 0.02)
    W, taps = z["width"], 4
    mlp = {"kind": "moe", "expert": {"ff": z["moe_ff"]}, "router": {"experts": z["experts"], "identity": z["identity"], "top": z["top"], "scale": 1.0},
           "shared": {"ff": z["shared"]}}
    rot = {"base": 10000.0, "dims": z["rot"], "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    lat = {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot"], "vdim": z["vdim"], "kv_rank": z["kv_rank"], "q_rank": z["q_rank"],
           "mask": {"size": z["window"]}, "rot": rot, "scale": (z["dim"] + z["rot"]) ** -0.5}
    gla = {"heads": z["gheads"], "dim": z["gdim"], "vdim": z["gvdim"], "tau": 16.0}
    layers = [{"type": "latent_attention", "mixer": lat, "mlp": mlp} if c == "l" else
              {"type": "latent_attention", "mixer": dict(lat, kv_from=z["order"].index("l")), "mlp": mlp} if c == "s" else
              {"type": "gla", "mixer": gla, "mlp": mlp} for c in z["order"]]
    cfg = {"architecture": "Fegizen", "width": W, "vocab": z["vocab"], "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0}, "canon": {"taps": taps},
           "logit_scale": 1.0, "layers": layers}
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    shapes = {"embed": (z["vocab"], W), "final.norm": (W,), "head": (z["vocab"], W)}
    EA = z["experts"] + z["identity"]
    for i, c in enumerate(z["order"]):
        p, m, f = "l%d." % i, "l%d.mix." % i, "l%d.mlp." % i
        shapes.update({p + "norm1": (W,), p + "norm2": (W,), p + "canon1": (W, taps), p + "canon2": (W, taps), p + "dwa": (i + 2,),
                       f + "router": (EA, W), f + "correction": (EA,), f + "shared.gate": (z["shared"], W), f + "shared.up": (z["shared"], W),
                       f + "shared.down": (W, z["shared"])})
        for e in range(z["experts"]):
            shapes.update({f + "e%d.gate" % e: (z["moe_ff"], W), f + "e%d.up" % e: (z["moe_ff"], W), f + "e%d.down" % e: (W, z["moe_ff"])})
        if c in "ls":
            H, no = z["heads"], z["heads"] * z["vdim"]
            shapes.update({m + "dq": (z["q_rank"], W), m + "dq.norm": (z["q_rank"],), m + "uq": (H * (z["dim"] + z["rot"]), z["q_rank"]),
                           m + "uk": (H * z["dim"], z["kv_rank"]), m + "uv": (no, z["kv_rank"]), m + "g": (no, W), m + "o": (W, no)})
            if c == "l":
                shapes.update({m + "dkv": (z["kv_rank"] + z["rot"], W), m + "dkv.norm": (z["kv_rank"],)})
        else:
            hd, hp = z["gheads"] * z["gdim"], z["gheads"] * z["gvdim"]
            shapes.update({m + "q": (hd, W), m + "k": (hd, W), m + "v": (hp, W), m + "g": (hp, W), m + "o": (W, hp), m + "norm": (z["gvdim"],),
                           m + "a1": (z["rank"], W), m + "a2": (hd, z["rank"]), m + "a2.b": (hd,)})
    header, off = {}, 0
    for name, shp in shapes.items():
        n = int(np.prod(shp))
        header[name] = {"dtype": "BF16", "shape": list(shp), "data_offsets": [off, off + 2 * n]}
        off += 2 * n
    h = json.dumps(header).encode()
    h += b" " * (-len(h) % 8)
    one, zero = _bf16(np.ones(1, np.float32))[0], np.uint16(0)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h)
        for k, (name, shp) in enumerate(shapes.items()):
            n = int(np.prod(shp))
            if name.endswith("norm") or name.endswith("norm1") or name.endswith("norm2"):
                f.write(np.full(n, one, np.uint16).tobytes())
            elif name.endswith(".dwa"):
                f.write(np.array([zero] * (n - 1) + [one], np.uint16).tobytes())
            elif len(shp) < 2:
                f.write(block[:n].tobytes())
            else:
                f.write(np.resize(np.roll(block, 7919 * k), n).tobytes())
    return cfg


def fegizen_numbers(z):
    """-> (decode bytes per token at CONTEXT, prefill FLOP per token): the active matrices once (bf16), the fp32 matrix states read
    and written, the window of cached rows (one row per position for all heads); 2 FLOP per active parameter plus the attention's
    and the recurrence's own products (queries against the cached rows: heads x (kv_rank + rot) per key, twice)."""
    W = z["width"]
    experts = z["top"] * 3 * z["moe_ff"] * W + (z["experts"] + z["identity"]) * W + 3 * z["shared"] * W
    params, state, extra = z["vocab"] * W, 0, 0.0
    seen = min(CONTEXT, z["window"])
    for c in z["order"]:
        if c in "ls":
            H, no, row = z["heads"], z["heads"] * z["vdim"], z["kv_rank"] + z["rot"]
            params += (z["q_rank"] + (row if c == "l" else 0) + 2 * no) * W + H * (z["dim"] + z["rot"]) * z["q_rank"] + H * z["dim"] * z["kv_rank"] + \
                no * z["kv_rank"] + experts
            state += seen * row * 2
            extra += 2.0 * H * seen * (row + z["kv_rank"])
        else:
            hd, hp = z["gheads"] * z["gdim"], z["gheads"] * z["gvdim"]
            params += (2 * hd + 2 * hp + z["rank"]) * W + z["rank"] * hd + hp * W + experts
            state += 2 * 4 * z["gheads"] * z["gdim"] * z["gvdim"]
            extra += 6.0 * z["gheads"] * z["gdim"] * z["gvdim"]
    return 2 * params + state, 2.0 * (params - z["vocab"] * W) + extra


def run_fegizen(args, base, emit, shm_path, ClockSampler):
    """`bench.py --workload fegizen-sizes`: the Fegizen design beside the closest existing model on the same executor, Fapudra
    (windowed attention + a matrix-state recurrence + routed experts), at equal width, heads, window, experts, layers and
    vocabulary."""
    import torch
    from yalm_b200 import api
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peaks = json.load(open(pk)) if os.path.exists(pk) else {"hbm_gbs": 6650.0, "bf16_tflops_sustained": 1400.0}
    hbm, tflops = float(peaks["hbm_gbs"]), float(peaks["bf16_tflops_sustained"])
    steps = max(8, min(args.steps, 128))
    clocks = ClockSampler(0)
    clocks.start()
    out, launches = [], 0

    def measure(model, ids):
        st = api.InferenceState(model)
        st.forward_batch(ids[:1024], 0)                     # warm-up (sizes kernels, first-use set-up)
        st.end_sequence()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        st.forward_batch(ids[:-1], 0)
        t_pre = time.perf_counter() - t0
        st.generate_greedy(ids[-1], CONTEXT - 1, max(3, args.warmup))   # first step eager + graph capture, untimed
        st.generate_greedy(ids[0], CONTEXT - 1 + max(3, args.warmup), steps)
        t_dec = st.device_ms / 1e3
        n = model.launches()
        st.close()
        return (CONTEXT - 1) / t_pre, steps / t_dec, n

    only = os.environ.get("YALM_BENCH_SIZES", "").split(",") if os.environ.get("YALM_BENCH_SIZES") else None
    for name, z in FEGIZEN_SIZES.items():
        if only and name not in only:
            continue
        ids = [(i * 7919 + 1) % z["vocab"] for i in range(CONTEXT)]
        row = {"size": name, "width": z["width"], "layers": z["order"], "context": CONTEXT, "window": z["window"]}
        folder = shm_path("yalm_bench_fegizen_%s_%d" % (name, os.getpid()))
        try:
            write_fegizen(folder, z)
            model = api.Model(folder, CONTEXT + steps + args.warmup + 8, api.BF16).cuda(0)
        finally:
            shutil.rmtree(folder, ignore_errors=True)
        pre, dec, n = measure(model, ids)
        model.close()
        dec_bytes, pre_flop = fegizen_numbers(z)
        launches += steps * n
        row["fegizen"] = {"prefill_tok_s": pre, "decode_tok_s": dec, "prefill_frac_of_measured_bf16": pre_flop * pre / 1e12 / tflops,
                          "decode_frac_of_measured_hbm": dec_bytes * dec / 1e9 / hbm, "decode_bytes_per_token": dec_bytes, "launches_per_token": n}
        if not os.environ.get("YALM_BENCH_NO_PEER"):
            zf = dict(FAPUDRA_SIZES[name])
            folder = shm_path("yalm_bench_fapudra_%s_%d" % (name, os.getpid()))
            try:
                write_fapudra(folder, zf, CONTEXT + steps + args.warmup + 8)
                model = api.Model(folder, 0, api.BF16).cuda(0)
            finally:
                shutil.rmtree(folder, ignore_errors=True)
            pre, dec, n = measure(model, ids)
            model.close()
            f_bytes, f_flop = fapudra_numbers(zf)
            row["equal_size_fapudra"] = {"prefill_tok_s": pre, "decode_tok_s": dec, "prefill_frac_of_measured_bf16": f_flop * pre / 1e12 / tflops,
                                         "decode_frac_of_measured_hbm": f_bytes * dec / 1e9 / hbm, "decode_bytes_per_token": f_bytes, "launches_per_token": n}
        out.append(row)
    clk = clocks.stop()
    first = out[0]["fegizen"]
    emit(dict(base, impl="ours", metric="batch-1 decode tok/s (Fegizen, first size; all sizes under `sizes`)", value=first["decode_tok_s"], steps=steps,
              ms_per_step=1000.0 / first["decode_tok_s"], dtype="bf16", clocks=clk, gpu_launches=launches, sizes=out,
              e2e={"value": first["decode_tok_s"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 4,
                   "note": "device loop: token ids stay on the device, 4 bytes per token come back"},
              config=dict(base["config"], workload="Fegizen at model-like sizes beside the equal-size Fapudra stack", context=CONTEXT,
                          l2="inputs larger than L2 (weights streamed per token)")))


# ---- Kiduvik ---------------------------------------------------------------------------------------------------------------
# name: width; latent attention heads x (dim unrotated + rot rotated), values, latent size; differential attention heads / kv heads of
# dim per map, values, window, kept first tokens; feed-forward (not gated), token side size; layer order (l = latent attention with its
# own cache, s = latent attention on the first l's cache, d = differential attention)
KIDUVIK_SIZES = {
    "w2048": dict(width=2048, heads=16, dim=64, rot=64, vdim=128, kv_rank=512, dheads=16, dkv=4, ddim=64, dvdim=128, window=1024, keep=4, ff=8192, side=64,
                  order="lsdl", vocab=32000),
    "w4096": dict(width=4096, heads=32, dim=64, rot=64, vdim=128, kv_rank=512, dheads=32, dkv=8, ddim=64, dvdim=128, window=2048, keep=4, ff=14336, side=64,
                  order="lds", vocab=32000),
}


def write_kiduvik(folder, z, context):
    """A checkpoint directory of the given size: matrices tiled from one random block, norm weights 1, sinks and lambda vectors small."""
    os.makedirs(folder, exist_ok=True)
    rng = np.random.default_rng(4)
    block = _bf16(rng.standard_normal(1 << 22).astype(np.float32) * 0.02)
    W, n_layers = z["width"], len(z["order"])
    mlp = {"kind": "dense", "ff": z["ff"]}
    lat = {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot"], "vdim": z["vdim"], "kv_rank": z["kv_rank"], "rot": {"base": 10000.0, "dims": z["rot"]},
           "scale": (z["dim"] + z["rot"]) ** -0.5}
    dif = {"heads": z["dheads"], "kv_heads": z["dkv"], "dim": z["ddim"], "vdim": z["dvdim"], "diff": 0.8, "mask": {"size": z["window"], "keep_first": z["keep"]},
           "rot": {"base": 500000.0, "dims": z["ddim"] // 2, "scaling": {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}}, "scale": z["ddim"] ** -0.5}
    layers = [{"type": "latent_attention", "mixer": lat, "mlp": mlp} if c == "l" else
              {"type": "latent_attention", "mixer": dict(lat, kv_from=z["order"].index("l")), "mlp": mlp} if c == "s" else
              {"type": "attention", "mixer": dif, "mlp": mlp} for c in z["order"]]
    cfg = {"architecture": "Kiduvik", "width": W, "vocab": z["vocab"], "max_positions": context, "norm": {"eps": 1e-5}, "token_side": {"dim": z["side"]},
           "layers": layers}
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    shapes = {"embed": (z["vocab"], W), "pos": (context, W), "side.embed": (z["vocab"], n_layers * z["side"]), "final.norm": (W,), "head": (z["vocab"], W)}
    for i, c in enumerate(z["order"]):
        p, m, f, sd = "l%d." % i, "l%d.mix." % i, "l%d.mlp." % i, "l%d.side." % i
        shapes.update({p + "norm1": (W,), p + "norm1b": (W,), p + "norm2": (W,), p + "norm2b": (W,), f + "up": (z["ff"], W), f + "down": (W, z["ff"]),
                       sd + "gate": (z["side"], W), sd + "proj": (W, z["side"]), sd + "norm": (W,)})
        if c in "ls":
            H, no = z["heads"], z["heads"] * z["vdim"]
            shapes.update({m + "q": (H * (z["dim"] + z["rot"]), W), m + "uk": (H * z["dim"], z["kv_rank"]), m + "uv": (no, z["kv_rank"]), m + "sink": (H,),
                           m + "o": (W, no)})
            if c == "l":
                shapes.update({m + "dkv": (z["kv_rank"] + z["rot"], W), m + "dkv.norm": (z["kv_rank"],)})
        else:
            H, G, D = z["dheads"], z["dkv"], z["ddim"]
            shapes.update({m + "q": (H * 2 * D, W), m + "k": (G * 2 * D, W), m + "v": (G * z["dvdim"], W), m + "q.norm": (D,), m + "k.norm": (D,),
                           m + "lq1": (D,), m + "lk1": (D,), m + "lq2": (D,), m + "lk2": (D,), m + "g": (H, W), m + "o": (W, H * z["dvdim"])})
    header, off = {}, 0
    for name, shp in shapes.items():
        n = int(np.prod(shp))
        header[name] = {"dtype": "BF16", "shape": list(shp), "data_offsets": [off, off + 2 * n]}
        off += 2 * n
    h = json.dumps(header).encode()
    h += b" " * (-len(h) % 8)
    one = _bf16(np.ones(1, np.float32))[0]
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h)
        for k, (name, shp) in enumerate(shapes.items()):
            n = int(np.prod(shp))
            last = name.split(".")[-1]
            if last.startswith("norm"):
                f.write(np.full(n, one, np.uint16).tobytes())
            elif len(shp) < 2:
                f.write(block[:n].tobytes())
            else:
                f.write(np.resize(np.roll(block, 7919 * k), n).tobytes())
    return cfg


def kiduvik_numbers(z):
    """-> (decode bytes per token at CONTEXT, prefill FLOP per token): every matrix once (bf16); per latent-attention layer one cached
    row per position for all heads over the whole context, per differential layer the window of both maps' keys and the values plus
    the kept first tokens; 2 FLOP per parameter plus the attention's own products (latent: heads x (kv_rank + rot) per key for the
    scores and kv_rank for the sums, over the causal half of the context on average in a prompt)."""
    W = z["width"]
    ffn = 2 * z["ff"] * W + 2 * z["side"] * W
    params, cache, extra = z["vocab"] * W, 0, 0.0
    for c in z["order"]:
        if c in "ls":
            H, no, row = z["heads"], z["heads"] * z["vdim"], z["kv_rank"] + z["rot"]
            params += (H * (z["dim"] + z["rot"]) + (row if c == "l" else 0) + no) * W + H * (z["dim"] + z["vdim"]) * z["kv_rank"] + ffn
            cache += CONTEXT * row * 2
            extra += 2.0 * H * (CONTEXT / 2) * (z["dim"] + z["rot"] + z["vdim"])
        else:
            H, G, D, dv = z["dheads"], z["dkv"], z["ddim"], z["dvdim"]
            seen = min(CONTEXT, z["window"])
            params += (2 * H * D + 2 * G * D + G * dv + H + H * dv) * W + ffn
            cache += seen * (2 * G * D + G * dv) * 2 + z["keep"] * (2 * G * D + G * dv) * 4
            extra += 2.0 * 2 * H * (seen + z["keep"]) * (D + dv)
    return 2 * params + cache, 2.0 * (params - z["vocab"] * W) + extra


def run_kiduvik(args, base, emit, shm_path, ClockSampler):
    """`bench.py --workload kiduvik-sizes`: the Kiduvik design beside the closest existing model on the same executor, the dense
    Retezen stack (windowed attention with pooled blocks, a norm on every sublayer's output, learned positions, dense feed-forward),
    at equal width, heads, head sizes, window, feed-forward size, layers and vocabulary."""
    import torch
    from yalm_b200 import api
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peaks = json.load(open(pk)) if os.path.exists(pk) else {"hbm_gbs": 6650.0, "bf16_tflops_sustained": 1400.0}
    hbm, tflops = float(peaks["hbm_gbs"]), float(peaks["bf16_tflops_sustained"])
    steps = max(8, min(args.steps, 128))
    clocks = ClockSampler(0)
    clocks.start()
    out, launches = [], 0

    def measure(model, ids):
        st = api.InferenceState(model)
        st.forward_batch(ids[:1024], 0)                     # warm-up (sizes kernels, first-use set-up)
        st.end_sequence()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        st.forward_batch(ids[:-1], 0)
        t_pre = time.perf_counter() - t0
        st.generate_greedy(ids[-1], CONTEXT - 1, max(3, args.warmup))   # first step eager + graph capture, untimed
        st.generate_greedy(ids[0], CONTEXT - 1 + max(3, args.warmup), steps)
        t_dec = st.device_ms / 1e3
        n = model.launches()
        st.close()
        return (CONTEXT - 1) / t_pre, steps / t_dec, n

    only = os.environ.get("YALM_BENCH_SIZES", "").split(",") if os.environ.get("YALM_BENCH_SIZES") else None
    for name, z in KIDUVIK_SIZES.items():
        if only and name not in only:
            continue
        ids = [(i * 7919 + 1) % z["vocab"] for i in range(CONTEXT)]
        row = {"size": name, "width": z["width"], "layers": z["order"], "context": CONTEXT, "window": z["window"]}
        folder = shm_path("yalm_bench_kiduvik_%s_%d" % (name, os.getpid()))
        try:
            write_kiduvik(folder, z, CONTEXT + steps + args.warmup + 8)
            model = api.Model(folder, 0, api.BF16).cuda(0)
        finally:
            shutil.rmtree(folder, ignore_errors=True)
        pre, dec, n = measure(model, ids)
        model.close()
        dec_bytes, pre_flop = kiduvik_numbers(z)
        launches += steps * n
        row["kiduvik"] = {"prefill_tok_s": pre, "decode_tok_s": dec, "prefill_frac_of_measured_bf16": pre_flop * pre / 1e12 / tflops,
                          "decode_frac_of_measured_hbm": dec_bytes * dec / 1e9 / hbm, "decode_bytes_per_token": dec_bytes, "launches_per_token": n}
        if not os.environ.get("YALM_BENCH_NO_PEER"):
            zr = dict(SIZES[name], layers=len(z["order"]))
            folder = shm_path("yalm_bench_retezen_peer_%s_%d" % (name, os.getpid()))
            try:
                write_retezen(folder, zr, "dense", CONTEXT + steps + args.warmup + 8)
                model = api.Model(folder, 0, api.BF16).cuda(0)
            finally:
                shutil.rmtree(folder, ignore_errors=True)
            pre, dec, n = measure(model, ids)
            model.close()
            _, r_bytes, r_flop = retezen_numbers(zr, "dense")
            row["equal_size_retezen"] = {"prefill_tok_s": pre, "decode_tok_s": dec, "prefill_frac_of_measured_bf16": r_flop * pre / 1e12 / tflops,
                                         "decode_frac_of_measured_hbm": r_bytes * dec / 1e9 / hbm, "decode_bytes_per_token": r_bytes, "launches_per_token": n}
        out.append(row)
    clk = clocks.stop()
    first = out[0]["kiduvik"]
    emit(dict(base, impl="ours", metric="batch-1 decode tok/s (Kiduvik, first size; all sizes under `sizes`)", value=first["decode_tok_s"], steps=steps,
              ms_per_step=1000.0 / first["decode_tok_s"], dtype="bf16", clocks=clk, gpu_launches=launches, sizes=out,
              e2e={"value": first["decode_tok_s"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 4,
                   "note": "device loop: token ids stay on the device, 4 bytes per token come back"},
              config=dict(base["config"], workload="Kiduvik at model-like sizes beside the equal-size dense Retezen stack", context=CONTEXT,
                          l2="inputs larger than L2 (weights streamed per token)")))


def run(args, base, emit, write_yalm, shm_path, ClockSampler):
    import torch
    from yalm_b200 import api
    from yalm_b200 import yalm_file as yf
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peaks = json.load(open(pk)) if os.path.exists(pk) else {"hbm_gbs": 6650.0, "bf16_tflops_sustained": 1400.0}
    hbm, tflops = float(peaks["hbm_gbs"]), float(peaks["bf16_tflops_sustained"])
    steps = max(8, min(args.steps, 128))
    clocks = ClockSampler(0)
    clocks.start()
    out, launches = [], 0
    for name, z in SIZES.items():
        for kind in ("dense", "moe"):
            ids = [(i * 7919 + 1) % z["vocab"] for i in range(CONTEXT)]
            row = {"size": name, "ffn": kind, "width": z["width"], "layers": z["layers"], "context": CONTEXT, "window": z["window"], "pool": z["pool"]}
            # ---- the new design ----
            folder = shm_path("yalm_bench_retezen_%s_%s_%d" % (name, kind, os.getpid()))
            try:
                write_retezen(folder, z, kind, CONTEXT + steps + args.warmup + 8)
                model = api.Model(folder, 0, api.BF16).cuda(0)
            finally:
                shutil.rmtree(folder, ignore_errors=True)
            st = api.InferenceState(model)
            st.forward_batch(ids[:1024], 0)                     # warm-up (sizes kernels, first-use set-up)
            st.end_sequence()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            st.forward_batch(ids[:-1], 0)
            t_pre = time.perf_counter() - t0
            st.generate_greedy(ids[-1], CONTEXT - 1, max(3, args.warmup))   # first step eager + graph capture, untimed
            pos = CONTEXT - 1 + max(3, args.warmup)
            st.generate_greedy(ids[0], pos, steps)
            t_dec = st.device_ms / 1e3
            params, dec_bytes, pre_flop = retezen_numbers(z, kind)
            launches += steps * model.launches()
            row["retezen"] = {"prefill_tok_s": (CONTEXT - 1) / t_pre, "decode_tok_s": steps / t_dec,
                              "prefill_frac_of_measured_bf16": pre_flop * (CONTEXT - 1) / t_pre / 1e12 / tflops,
                              "decode_frac_of_measured_hbm": dec_bytes * steps / t_dec / 1e9 / hbm, "decode_bytes_per_token": dec_bytes,
                              "launches_per_token": model.launches()}
            st.close()
            model.close()
            # ---- the closest existing model at equal size: the .yalm Llama / Mixtral block, fp16 ----
            arch = yf.Arch(z["width"], z["ff"] if kind == "dense" else z["moe_ff"], z["dim"], z["layers"], z["heads"], z["kv_heads"], z["vocab"],
                           CONTEXT + 256, 10000.0, n_experts=z["experts"] if kind == "moe" else 0, n_experts_active=z["top"] if kind == "moe" else 0,
                           name="equal-size-%s-%s" % (name, kind))
            path = shm_path("yalm_bench_equal_%s_%s_%d.yalm" % (name, kind, os.getpid()))
            write_yalm(path, arch, "fp16")
            try:
                model = api.Model(path, CONTEXT + 256).cuda(0)
            finally:
                os.unlink(path)
            st = api.InferenceState(model)
            cap = model.batch_capacity()
            ref = {"whole_token_kernel": model.uses_megakernel(), "launches_per_token": model.launches()}
            if cap:
                st.forward_batch(ids[:cap], 0)
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for p in range(0, CONTEXT - 1, cap):
                    st.forward_batch(ids[p:min(p + cap, CONTEXT - 1)], p)
                ref["prefill_tok_s"] = (CONTEXT - 1) / (time.perf_counter() - t0)
            else:                                               # no batched pass for this model: the token loop hydrates
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for p in range(256):
                    st.forward(ids[p], p, api.MODE_HYDRATE)
                torch.cuda.synchronize()
                ref["prefill_tok_s"] = 256 / (time.perf_counter() - t0)
                ref["prefill_note"] = "token loop (this model has no batched pass)"
                for p in range(256, CONTEXT - 1, 1):            # fill the context for the decode measurement
                    st.forward(ids[p], p, api.MODE_HYDRATE)
            st.generate_greedy(ids[-1], CONTEXT - 1, max(3, args.warmup))
            st.generate_greedy(ids[0], CONTEXT - 1 + max(3, args.warmup), steps)
            ref["decode_tok_s"] = steps / (st.device_ms / 1e3)
            full_kv = z["layers"] * CONTEXT * 2 * z["kv_heads"] * z["dim"] * 2
            ref["decode_frac_of_measured_hbm"] = (2 * params + full_kv) * ref["decode_tok_s"] / 1e9 / hbm
            ref["prefill_frac_of_measured_bf16"] = (2.0 * (params - z["vocab"] * z["width"]) + 4.0 * z["layers"] * z["heads"] * z["dim"] * CONTEXT / 2) * \
                ref["prefill_tok_s"] / 1e12 / tflops
            row["equal_size_yalm"] = ref
            st.close()
            model.close()
            # ---- the same model on its per-op kernels (one launch per product, as the layered executor has): the like-for-like
            # reading of the one-row products, which are the same streaming GEMV in both ----
            os.environ["YALM_B200_MEGA"] = "0"
            try:
                write_yalm(path, arch, "fp16")
                try:
                    model = api.Model(path, CONTEXT + 256).cuda(0)
                finally:
                    os.unlink(path)
                st = api.InferenceState(model)
                if cap:
                    for p in range(0, CONTEXT - 1, cap):
                        st.forward_batch(ids[p:min(p + cap, CONTEXT - 1)], p)
                else:
                    for p in range(CONTEXT - 1):
                        st.forward(ids[p], p, api.MODE_HYDRATE)
                st.generate_greedy(ids[-1], CONTEXT - 1, max(3, args.warmup))
                st.generate_greedy(ids[0], CONTEXT - 1 + max(3, args.warmup), steps)
                tok_s = steps / (st.device_ms / 1e3)
                ref["per_op_kernels"] = {"whole_token_kernel": model.uses_megakernel(), "launches_per_token": model.launches(), "decode_tok_s": tok_s,
                                         "decode_frac_of_measured_hbm": (2 * params + full_kv) * tok_s / 1e9 / hbm}
                st.close()
                model.close()
            finally:
                del os.environ["YALM_B200_MEGA"]
            out.append(row)
    clk = clocks.stop()
    first = out[0]["retezen"]
    emit(dict(base, impl="ours", metric="batch-1 decode tok/s (Retezen, first size; all sizes under `sizes`)", value=first["decode_tok_s"], steps=steps,
              ms_per_step=1000.0 / first["decode_tok_s"], dtype="bf16", clocks=clk, gpu_launches=launches, sizes=out,
              e2e={"value": first["decode_tok_s"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 4,
                   "note": "device loop: token ids stay on the device, 4 bytes per token come back"},
              config=dict(base["config"], workload="Retezen at model-like sizes beside the equal-size .yalm block", context=CONTEXT,
                          l2="inputs larger than L2 (weights streamed per token)")))
