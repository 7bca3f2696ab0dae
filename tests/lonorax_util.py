"""Small Lonorax models for the tests: configurations, random weights, a model folder. Weights are drawn in float64,
rounded to bfloat16, and both the file and the plain implementation get the rounded values, so that the two compute from
the same numbers. ``zurerax_util.run_schedule`` drives an engine for these models too."""
import json
import os

import numpy as np
import torch

from glassbox_b200.weights.safetensors_io import write_safetensors


def moe(experts, top, ff, groups=None, scale=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        router["scale"] = scale
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        mlp["shared"] = {"ff": shared}
    return mlp


def gru(width, mlp=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def attn(heads, kv_heads, dim, vdim, window=None, rot=None, scale=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def config(vocab, width, layers, streams=None, eps=1e-6):
    cfg = {"architecture": "Lonorax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        cfg["streams"] = streams
    return cfg


CONFIGS = {
    # nothing a power of two; three streams; value size unlike key size; a layer without a feed-forward; windows shorter
    # and longer than a page; rotation of a part and of the whole head; groups of two and of four; attention first
    "odd": lambda: config(203, 56, [
        attn(6, 2, 20, 12, window=7, rot=(8, 500.0), mlp=moe(6, 2, 24, groups=(3, 2), scale=2.5, shared=40)),
        gru(44),
        attn(4, 4, 16, 24, window=19, rot=(16, 10000.0), mlp=moe(8, 3, 16, groups=(2, 1))),
        gru(72, mlp=moe(5, 1, 20, shared=12)),
    ], streams=3, eps=1e-5),
    # sizes the vector loads and the tensor-core products are built for; two streams; a window of 33 (a page border plus one)
    "even": lambda: config(320, 128, [
        gru(256, mlp=moe(8, 2, 64, groups=(4, 2), scale=1.0, shared=128)),
        attn(8, 2, 64, 64, window=33, rot=(32, 20000.0), mlp=moe(16, 4, 32, groups=(4, 3), scale=0.5, shared=64)),
        gru(128, mlp=None),
        attn(4, 1, 128, 32, window=48, rot=(64, 1e6), scale=0.2, mlp=moe(4, 2, 128, scale=1.5)),
    ], streams=2),
    # what the design lets a model leave out: one plain residual row, no window, no rotation, no groups, no shared expert
    "plain": lambda: config(97, 48, [
        attn(3, 1, 16, 16, mlp=moe(4, 2, 24)),
        gru(40, mlp=moe(3, 3, 16, scale=0.7)),
        attn(2, 2, 8, 24, rot=(4, 100.0), mlp=None),
    ]),
    # ones: one stream, one head, a window of one token (a position sees itself alone), one expert, groups of one expert
    "ones": lambda: config(61, 32, [
        attn(1, 1, 8, 8, window=1, rot=(2, 10.0), mlp=moe(1, 1, 8)),
        gru(1, mlp=moe(4, 1, 8, groups=(4, 2), shared=8)),
        attn(2, 1, 8, 8, window=2, mlp=None),
    ], streams=1),
    # sizes that fit no vector width: odd row lengths everywhere, so every kernel's aligned fast path must step aside
    "ragged": lambda: config(67, 50, [
        gru(13, mlp=moe(3, 2, 11, shared=7)),
        attn(3, 1, 10, 7, window=5, rot=(6, 300.0), mlp=moe(6, 2, 9, groups=(2, 1), scale=1.3)),
    ], streams=5),
}


def tensor_shapes(cfg):
    d, S = cfg["width"], cfg.get("streams")
    shapes = {"embed": (cfg["vocab"], d), "final.norm": (d,), "final.norm.b": (d,), "head": (cfg["vocab"], d)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for q in (1, 2) if L["mlp"] is not None else (1,):
            shapes[p + f"norm{q}"] = shapes[p + f"norm{q}.b"] = (d,)
            if S:
                shapes.update({p + f"hc{q}.in": (S,), p + f"hc{q}.out": (S,), p + f"hc{q}.mix": (S, S)})
        if L["type"] == "mingru":
            w = m["width"]
            shapes.update({p + "mix.z": (w, d), p + "mix.z.b": (w,), p + "mix.x": (w, d), p + "mix.x.b": (w,),
                           p + "mix.g": (w, d), p + "mix.o": (d, w)})
        else:
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (H * D, d), p + "mix.k": (G * D, d), p + "mix.v": (G * V, d), p + "mix.q.norm": (D,),
                           p + "mix.k.norm": (D,), p + "mix.pb": (H,), p + "mix.o": (d, H * V)})
        if L["mlp"] is not None:
            f, r = L["mlp"], L["mlp"]["router"]
            shapes.update({p + "mlp.router": (r["experts"], d), p + "mlp.correction": (r["experts"],)})
            for e in range(r["experts"]):
                shapes.update({p + f"mlp.e{e}.up": (f["expert"]["ff"], d), p + f"mlp.e{e}.down": (d, f["expert"]["ff"])})
            if f.get("shared") is not None:
                shapes.update({p + "mlp.shared.up": (f["shared"]["ff"], d), p + "mlp.shared.down": (d, f["shared"]["ff"]),
                               p + "mlp.shared.sg": (1, d)})
    return shapes


def _bf16(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16)


def random_weights(cfg, seed):
    """{name: bfloat16 tensor}. Matrices are N(0, 1/in), so that every projection of a normed row is of order one; the
    streams' mixing is the identity plus noise, their read weights sum to about one; gate biases lean towards keeping the
    state, head biases towards small weights, corrections are large enough to change who is chosen."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if name.endswith("mlp.router"):
            w = rng.standard_normal(shape) * 2.0 / np.sqrt(shape[1])
        elif name.endswith("hc1.mix") or name.endswith("hc2.mix"):
            w = np.eye(shape[0]) + rng.standard_normal(shape) * 0.15
        elif len(shape) == 2:
            w = rng.standard_normal(shape) / np.sqrt(shape[1])
        elif leaf == "in":
            w = 1.0 / shape[0] + rng.standard_normal(shape) * 0.2
        elif leaf == "out":
            w = 1.0 + rng.standard_normal(shape) * 0.2
        elif name.endswith("z.b"):
            w = rng.standard_normal(shape) * 1.5 - 1.0
        elif name.endswith("x.b"):
            w = rng.standard_normal(shape) * 0.3
        elif leaf == "pb":
            w = rng.standard_normal(shape) * 0.5 - 1.5
        elif leaf == "correction":
            w = rng.standard_normal(shape) * 0.4 - 0.6          # (choice scores around zero: negative ones occur)
        elif leaf == "b":
            w = rng.standard_normal(shape) * 0.1
        elif leaf in ("norm1", "norm2", "norm"):
            w = 1.0 + rng.standard_normal(shape) * 0.2
        else:
            raise AssertionError(name)
        out[name] = _bf16(w)
    return out


def as_float64(tensors):
    return {k: v.float().numpy().astype(np.float64) for k, v in tensors.items()}


def write_model(folder, cfg, tensors):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {k: v.contiguous() for k, v in tensors.items()})
    return folder
