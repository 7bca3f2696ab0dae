"""Small Zurerax models for the tests: configurations, random (or crafted) weights, a model folder, and helpers that
run requests through an engine under a schedule. Weights are drawn in float64, rounded to bfloat16, and both the file and
the plain implementation get the rounded values, so that the two compute from the same numbers."""
import json
import os

import numpy as np
import torch

from glassbox_b200.weights.safetensors_io import write_safetensors


def delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank, mlp=None):
    return {"type": "channel_delta", "mlp": {"kind": "dense", "ff": mlp} if mlp else None,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                      "decay_rank": decay_rank, "gate_rank": gate_rank}}


def latent(heads, dim, rot_dim, vdim, kv_rank, base=10000.0, scale=None, kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "rot": {"base": base, "dims": rot_dim}, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mlp": {"kind": "dense", "ff": mlp} if mlp else None, "mixer": m}


def config(vocab, width, layers, embedding_scale=1.0, logit_scale=1.0, eps=1e-6):
    return {"architecture": "Zurerax", "vocab": vocab, "width": width, "embedding": {"scale": embedding_scale},
            "logit_scale": logit_scale, "norm": {"eps": eps}, "layers": layers}


CONFIGS = {
    # nothing a power of two; grouped key heads; a layer without a feed-forward; a layer that reads another's cache;
    # attention first and last
    "odd": lambda: config(211, 72, [
        latent(3, 24, 8, 20, 40, base=1000.0, mlp=100),
        delta(4, 2, 24, 20, 3, 5, 7, mlp=None),
        latent(2, 16, 8, 12, 40, base=1000.0, kv_from=0, mlp=52),
        delta(2, 2, 16, 48, 2, 3, 4, mlp=36),
        latent(1, 8, 4, 8, 16, base=50.0, mlp=None),
    ], embedding_scale=3.0, logit_scale=0.7, eps=1e-5),
    # sizes the tensor-core kernels are built for; two readers of one cache; five taps; one key head for all value heads
    "even": lambda: config(320, 128, [
        delta(4, 1, 32, 64, 5, 8, 8, mlp=256),
        latent(8, 32, 16, 32, 64, base=20000.0, mlp=256),
        latent(4, 64, 16, 64, 64, base=20000.0, kv_from=1, mlp=None),
        latent(16, 16, 16, 16, 64, base=20000.0, kv_from=1, mlp=128),
        delta(2, 2, 128, 32, 4, 16, 4, mlp=128),
    ], embedding_scale=11.3, logit_scale=2.5),
    # sizes that fit no vector width: odd row lengths everywhere, so every kernel's aligned fast path must step aside
    "ragged": lambda: config(67, 50, [
        latent(3, 10, 6, 7, 9, base=300.0, mlp=30),
        delta(3, 1, 10, 7, 3, 3, 5, mlp=None),
        latent(5, 6, 6, 3, 9, base=300.0, kv_from=0, mlp=22),
    ], embedding_scale=2.0, logit_scale=1.3),
    # ones: one head, one tap (no convolution state), rank one, no feed-forward anywhere
    "ones": lambda: config(97, 40, [
        delta(1, 1, 8, 8, 1, 1, 1),
        latent(1, 8, 2, 8, 8, base=7.0),
    ]),
}


def tensor_shapes(cfg):
    d, shapes = cfg["width"], {"embed": (cfg["vocab"], cfg["width"]), "final.norm": (cfg["width"],),
                               "head": (cfg["vocab"], cfg["width"])}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1b"] = (d,)
        if L["type"] == "channel_delta":
            H, KH, D, V, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            shapes.update({p + "mix.q": (KH * D, d), p + "mix.k": (KH * D, d), p + "mix.v": (H * V, d),
                           p + "mix.q.conv": (KH * D, taps), p + "mix.k.conv": (KH * D, taps), p + "mix.v.conv": (H * V, taps),
                           p + "mix.b": (H, d), p + "mix.A_log": (H,), p + "mix.norm": (V,),
                           p + "mix.a1": (m["decay_rank"], d), p + "mix.a2": (H * D, m["decay_rank"]), p + "mix.dt_bias": (H * D,),
                           p + "mix.g1": (m["gate_rank"], d), p + "mix.g2": (H * V, m["gate_rank"]), p + "mix.o": (d, H * V)})
        else:
            H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            shapes.update({p + "mix.q": (H * (D + R), d), p + "mix.uk": (H * D, C), p + "mix.uv": (H * V, C),
                           p + "mix.sink": (H,), p + "mix.o": (d, H * V)})
            if "kv_from" not in m:
                shapes.update({p + "mix.dkv": (C + R, d), p + "mix.dkv.norm": (C,)})
        if L["mlp"] is not None:
            shapes.update({p + "norm2": (d,), p + "norm2b": (d,), p + "mlp.up": (L["mlp"]["ff"], d),
                           p + "mlp.down": (d, L["mlp"]["ff"])})
    return shapes


def _bf16(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16)


def random_weights(cfg, seed, sharpen=1.0):
    """{name: bfloat16 tensor}. Matrices are N(0, 1/in) so that every projection of a unit-RMS row is of order one;
    ``sharpen`` multiplies the query projections, so that a few keys carry each softmax."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if len(shape) == 2 and not name.endswith(".conv"):
            w = rng.standard_normal(shape) / np.sqrt(shape[1])
            if name.endswith("mix.q") and f"{name[:-1]}uk" in tensor_shapes(cfg):
                w *= sharpen
        elif name.endswith(".conv"):
            w = rng.standard_normal(shape) * 0.6
        elif leaf in ("norm1", "norm1b", "norm2", "norm2b") or name == "final.norm":
            w = rng.standard_normal(shape) * 0.2               # stored around zero
        elif leaf == "norm":                                   # (dkv.norm and the read-out norm: plain gains)
            w = 1.0 + rng.standard_normal(shape) * 0.2
        elif leaf == "A_log":
            w = rng.uniform(-2.0, 0.5, shape)
        elif leaf == "dt_bias":
            w = rng.standard_normal(shape)
        elif leaf == "sink":
            w = rng.standard_normal(shape) * 1.5
        else:
            raise AssertionError(name)
        out[name] = _bf16(w)
    return out


def as_float64(tensors):
    return {k: v.float().numpy().astype(np.float64) for k, v in tensors.items()}


def file_config(cfg):
    """The config as a weights folder holds it: the ranks are in no key, only in the shapes."""
    out = json.loads(json.dumps(cfg))
    for L in out["layers"]:
        L["mixer"].pop("decay_rank", None)
        L["mixer"].pop("gate_rank", None)
    return out


def write_model(folder, cfg, tensors):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(file_config(cfg), f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {k: v.contiguous() for k, v in tensors.items()})
    return folder


def run_schedule(engine, requests, schedule):
    """``requests``: {id: tokens}; ``schedule``: a list of steps, each a list of (id, count). Every position's logits are
    asked for. A request is admitted at its first entry and freed after its last token. Returns {id: float32 [T, vocab]}."""
    from glassbox_b200.engine.engine import StepEntry
    at = {rid: 0 for rid in requests}
    got = {rid: [] for rid in requests}
    for step in schedule:
        entries = []
        for rid, count in step:
            if at[rid] == 0:
                engine.add_request(rid, [])
            entries.append(StepEntry(rid, requests[rid][at[rid]:at[rid] + count], list(range(count))))
        logits = engine.step(entries).float().cpu().numpy()
        engine.check()
        row = 0
        for rid, count in step:
            got[rid].append(logits[row:row + count].copy())
            row += count
            at[rid] += count
            if at[rid] == len(requests[rid]):
                engine.free_request(rid)
    assert all(at[r] == len(requests[r]) for r in requests), "the schedule does not cover every request"
    return {rid: np.concatenate(v, 0) for rid, v in got.items()}
