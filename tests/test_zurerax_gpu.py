"""Zurerax on the GPU against the plain float64 implementation (``tests/plain/zurerax_plain.py``): each mechanism's
kernel alone, then whole models under every way of cutting and batching their requests, through the engine's own step
function, cache manager, scheduler and entry point. Sizes are the tests' own (``zurerax_util.CONFIGS``)."""
import numpy as np
import pytest
import torch

import conftest
from plain import zurerax_plain as plain
import zurerax_util as zu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# bfloat16: a layer here rounds an activation about a dozen times (two norms in, two branch norms out, three products and
# an activation in the feed-forward, five or more in a mixer) and every branch is normed back to unit size before it
# joins the residual, so a rounding error of 2^-9 keeps its relative size through the layer; five layers give a mean
# error of about sqrt(60) * 2^-9 = 1.5 % of the logits' spread (single logits of the tiniest models, whose norms run over eight numbers, stray further: measured up to 0.2). Faults in which key or state a bfloat16 kernel reads are caught by the crafted test above and by the float32 runs of the same code. float32 keeps the suite's absolute bound.
BF16_REL_MAX, BF16_REL_MEAN = 0.25, 0.02


def assert_logits_close(got, want, dtype, what=""):
    if dtype == "float32":
        return conftest.assert_logits_close(got, want, dtype, what)
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    diff, spread = np.abs(got - want), want.std()
    assert diff.max() <= BF16_REL_MAX * spread, f"{what}: max abs diff {diff.max():.3e} > {BF16_REL_MAX} x spread {spread:.3e}"
    assert diff.mean() <= BF16_REL_MEAN * spread, f"{what}: mean abs diff {diff.mean():.3e} > {BF16_REL_MEAN} x spread {spread:.3e}"


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def _steps_meta(portions, slots):
    """Device metadata of one step: ``portions`` [(start position, rows) or None for a padding sequence]."""
    row_seq, positions, first, start = [], [], [], []
    row = 0
    for s, p in enumerate(portions):
        first.append(row)
        if p is None:
            start.append(-1); row_seq.append(s); positions.append(-1); row += 1
            continue
        start.append(p[0])
        for i in range(p[1]):
            row_seq.append(s); positions.append(p[0] + i)
        row += p[1]
    first.append(row)
    return dict(n=row, row_seq=_i32(row_seq), positions=_i32(positions), first=_i32(first), start=_i32(start), slots=_i32(slots))


# ------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("taps", [1, 2, 4, 5])
def test_short_conv_carries_its_last_inputs(taps):
    from glassbox_b200 import kernels
    rng = np.random.default_rng(taps)
    C, lens = 37, {"a": 13, "b": 9}
    x = {k: rng.standard_normal((n, C)) for k, n in lens.items()}
    w = rng.standard_normal((C, taps))
    want = {k: plain.silu(plain.causal_conv(x[k], w)) for k in x}
    state = torch.full((3, 11 + (taps - 1) * C), 7.0, device=DEV)      # slot 1 is nobody's and must stay as it is
    state[0].zero_(); state[2].zero_()
    slot = {"a": 2, "b": 0}
    # portions of 1, 2 and more rows, shorter and longer than the taps; a padding sequence in between
    plan = [[("a", 1), None, ("b", 4)], [("b", 1), ("a", 2)], [("a", 7), ("b", 2)], [("b", 2), None, ("a", 3)]]
    at, got = {"a": 0, "b": 0}, {"a": [], "b": []}
    wt = torch.tensor(w, dtype=torch.float32, device=DEV)
    for step in plan:
        portions = [None if e is None else (at[e[0]], e[1]) for e in step]
        meta = _steps_meta(portions, [0 if e is None else slot[e[0]] for e in step])
        rows = [np.zeros((1, C)) if e is None else x[e[0]][at[e[0]]:at[e[0]] + e[1]] for e in step]
        xin = torch.tensor(np.concatenate(rows), dtype=torch.float32, device=DEV)
        y = torch.zeros_like(xin)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        kernels.short_conv(xin, wt, y, state, 11, meta["row_seq"], meta["positions"], meta["first"], meta["start"],
                           meta["slots"], True, status)
        assert int(status.item()) == 0
        row = 0
        for e in step:
            if e is None:
                row += 1
                continue
            got[e[0]].append(y[row:row + e[1]].cpu().numpy())
            row += e[1]
            at[e[0]] += e[1]
    for k in x:
        np.testing.assert_allclose(np.concatenate(got[k]), want[k], atol=2e-5)
    assert torch.all(state[1] == 7.0) and torch.all(state[:, :11][[0, 2]] == 0)


@pytest.mark.parametrize("H, KH, D, V", [(4, 2, 24, 20), (2, 2, 64, 32), (1, 1, 160, 8), (2, 1, 8, 130), (3, 3, 128, 64)])
def test_delta_rule_kernel(H, KH, D, V):
    from glassbox_b200 import kernels
    rng = np.random.default_rng(D + V)
    lens = [21, 1, 6]
    cuts = [[17, 4], [1], [2, 4]]                                   # each sequence in two steps (or one)
    qkv = [rng.standard_normal((n, 2 * KH * D + H * V)) for n in lens]
    beta = [rng.standard_normal((n, H)) * 2 for n in lens]
    a = [rng.standard_normal((n, H * D)) * 2 for n in lens]
    dt_bias, a_log = rng.standard_normal(H * D), rng.uniform(-2, 0.5, H)
    want = []
    for s, n in enumerate(lens):
        q = qkv[s][:, :KH * D].reshape(n, KH, D)
        k = qkv[s][:, KH * D:2 * KH * D].reshape(n, KH, D)
        q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
        k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
        q, k = np.repeat(q, H // KH, 1), np.repeat(k, H // KH, 1)
        g = np.exp(-np.exp(a_log)[None, :, None] * plain.softplus(a[s] + dt_bias).reshape(n, H, D))
        want.append(plain.delta_rule(q, k, qkv[s][:, 2 * KH * D:].reshape(n, H, V), g, plain.sigmoid(beta[s])).reshape(n, H * V))
    f = lambda arr: torch.tensor(arr, dtype=torch.float32, device=DEV)
    state = torch.zeros((4, H * D * V + 5), device=DEV)
    state[1] = 3.0                                                  # a slot that belongs to nobody
    slots = [3, 0, 2]
    got = [[] for _ in lens]
    at = [0, 0, 0]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for step in range(2):
        live = [s for s in range(3) if step < len(cuts[s])]
        portions, sl = [], []
        for s in live:
            portions.append((at[s], cuts[s][step])); sl.append(slots[s])
            if s == 0:
                portions.append(None); sl.append(0)               # a padding sequence right behind a real one
        meta = _steps_meta(portions, sl)
        order = []                                                  # (sequence, None for the padding row behind it)
        for s in live:
            order.append((s, 1))
            if s == 0:
                order.append((s, None))

        def pick(arrs, width):
            return np.concatenate([arrs[s][at[s]:at[s] + cuts[s][step]] if tag is not None else np.zeros((1, width))
                                   for s, tag in order])
        out = torch.zeros((meta["n"], H * V), device=DEV)
        kernels.channel_delta(f(pick(qkv, 2 * KH * D + H * V)), f(pick(beta, H)), f(pick(a, H * D)), f(dt_bias), f(a_log), state, out,
                              meta["first"], meta["start"], meta["slots"], H, KH, D, V, True, status)
        row = 0
        for s, tag in order:
            if tag is None:
                row += 1
                continue
            got[s].append(out[row:row + cuts[s][step]].cpu().numpy())
            row += cuts[s][step]
        for s in live:
            at[s] += cuts[s][step]
    assert int(status.item()) == 0
    for s in range(3):
        np.testing.assert_allclose(np.concatenate(got[s]), want[s], atol=3e-5, rtol=1e-4)
    assert torch.all(state[1] == 3.0) and torch.all(state[:, H * D * V:][[0, 2, 3]] == 0)


@pytest.mark.parametrize("H, KH, D, V", [(4, 2, 24, 20), (2, 2, 128, 128), (3, 1, 64, 100)])
def test_delta_rule_kernel_for_single_tokens(H, KH, D, V):
    """The decoding form (one token per request and step, norm and gate in the same kernel) against the plain recurrence,
    several requests side by side, a padding request among them, the state carried from step to step."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(D * V)
    B, T = 3, 7
    qkv = rng.standard_normal((B, T, 2 * KH * D + H * V))
    beta, a, gate = rng.standard_normal((B, T, H)) * 2, rng.standard_normal((B, T, H * D)) * 2, rng.standard_normal((B, T, H * V))
    dt_bias, a_log, w = rng.standard_normal(H * D), rng.uniform(-2, 0.5, H), rng.standard_normal(V)
    f = lambda arr: torch.tensor(arr, dtype=torch.float32, device=DEV)
    state = torch.zeros((5, H * D * V + 3), device=DEV)
    state[4] = 2.0
    slots = [3, 0, 2]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = np.zeros((B, T, H * V))
    for t in range(T):
        # requests 0, 1, padding, 2
        meta = _steps_meta([(t, 1), (t, 1), None, (t, 1)], [slots[0], slots[1], 0, slots[2]])
        rows = [0, 1, None, 2]
        pick = lambda arr, width: np.stack([arr[b, t] if b is not None else np.zeros(width) for b in rows])
        att = torch.zeros((4, H * V), device=DEV)
        kernels.channel_delta_decode(f(pick(qkv, qkv.shape[-1])), f(pick(beta, H)), f(pick(a, H * D)), f(dt_bias), f(a_log), state,
                                     f(pick(gate, H * V)), f(w), 1e-5, att, meta["first"], meta["start"], meta["slots"], H, KH, D, V,
                                     True, status)
        out = att.cpu().numpy()
        got[0, t], got[1, t], got[2, t] = out[0], out[1], out[3]
        assert np.all(out[2] == 0)
    assert int(status.item()) == 0
    for b in range(B):
        q = qkv[b][:, :KH * D].reshape(T, KH, D)
        k = qkv[b][:, KH * D:2 * KH * D].reshape(T, KH, D)
        q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
        k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
        q, k = np.repeat(q, H // KH, 1), np.repeat(k, H // KH, 1)
        g = np.exp(-np.exp(a_log)[None, :, None] * plain.softplus(a[b] + dt_bias).reshape(T, H, D))
        o = plain.delta_rule(q, k, qkv[b][:, 2 * KH * D:].reshape(T, H, V), g, plain.sigmoid(beta[b]))
        want = (plain.rms_unit(o, 1e-5) * w * plain.sigmoid(gate[b].reshape(T, H, V))).reshape(T, H * V)
        np.testing.assert_allclose(got[b], want, atol=5e-5, rtol=2e-4)
    assert torch.all(state[4] == 2.0) and torch.all(state[1] == 0)


def test_branch_norm_head_norm_activation_and_scales():
    from glassbox_b200 import kernels
    rng = np.random.default_rng(9)
    n, d, H, V = 5, 72, 3, 20
    y, x, gain = rng.standard_normal((n, d)), rng.standard_normal((n, d)), rng.standard_normal(d)
    f = lambda arr: torch.tensor(arr, dtype=torch.float32, device=DEV)
    xt = f(x)
    kernels.rmsnorm_add(f(y), f(gain), xt, 1e-5)
    np.testing.assert_allclose(xt.cpu().numpy(), x + plain.rms_unit(y, 1e-5) * gain, atol=1e-5)
    o, gate, w = rng.standard_normal((n, H * V)), rng.standard_normal((n, H * V + 3)), rng.standard_normal(V)
    out = torch.zeros((n, H * V), device=DEV)
    kernels.gated_head_norm(f(o), f(gate)[:, 3:], f(w), out, H, 1e-6)
    want = (plain.rms_unit(o.reshape(n, H, V), 1e-6) * w * plain.sigmoid(gate[:, 3:].reshape(n, H, V))).reshape(n, H * V)
    np.testing.assert_allclose(out.cpu().numpy(), want, atol=1e-5)
    h = f(rng.standard_normal((n, 33)))
    act = torch.empty_like(h)
    kernels.relu2(h, act)
    assert torch.equal(act, torch.clamp(h, min=0) ** 2)
    table = torch.tensor(rng.standard_normal((11, 8)), dtype=torch.bfloat16, device=DEV)
    emb = torch.zeros((3, 8), device=DEV)
    kernels.embed(table, _i32([4, 0, 10]), emb, torch.zeros(1, dtype=torch.int32, device=DEV), scale=1.75)
    assert torch.equal(emb, table[[4, 0, 10]].float() * 1.75)
    kernels.scale_(emb, -0.5)
    assert torch.equal(emb, table[[4, 0, 10]].float() * 1.75 * -0.5)


@pytest.mark.parametrize("n, heads, N, K", [(1, 3, 40, 16), (70, 6, 128, 64), (200, 16, 64, 128), (33, 2, 130, 256)])
def test_one_small_product_per_head(n, heads, N, K):
    from glassbox_b200 import kernels
    g = torch.Generator(device="cpu").manual_seed(n)
    a_head, c_head = K + 8, N + 6
    a = torch.randn((n, heads * a_head), generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn((heads, N, K), generator=g) / K ** 0.5).to(torch.bfloat16).to(DEV)
    out = torch.full((n, heads * c_head), 9.0, dtype=torch.bfloat16, device=DEV)
    assert kernels.head_linear_supported(a, w, out, a_head, c_head)
    kernels.head_linear(a, w, out, a_head, c_head)
    a3 = a.float().view(n, heads, a_head)[:, :, :K]
    want = torch.einsum("nhk,hck->nhc", a3, w.float())
    got = out.float().view(n, heads, c_head)
    assert torch.allclose(got[:, :, :N], want, atol=0.03, rtol=0.02)
    assert torch.all(got[:, :, N:] == 9.0)                          # columns between the heads' outputs are not touched


def test_squared_relu_in_the_products_epilogue():
    from glassbox_b200 import kernels
    g = torch.Generator(device="cpu").manual_seed(3)
    for rows in (5, 200):
        a = torch.randn((rows, 128), generator=g).to(torch.bfloat16).to(DEV)
        w = (torch.randn((272, 128), generator=g) / 11).to(torch.bfloat16).to(DEV)
        want = torch.clamp(a.float() @ w.float().T, min=0) ** 2
        got = torch.zeros((rows, 272), dtype=torch.bfloat16, device=DEV)
        if rows <= kernels.STREAM_MAX_ROWS:
            kernels.gemm_stream(a, w, got, relu2=True)
        else:
            kernels.gemm_tc(a, w, got, relu2=True)
        assert torch.allclose(got.float(), want, atol=0.02, rtol=0.02), rows


def _run_latent_kernel(how, q, cache, table, lengths, sink, H, c, r, page):
    """q [n, H, c + r] for n requests that each bring their last token (request i holds ``lengths[i]`` tokens)."""
    from glassbox_b200 import kernels
    n = q.shape[0]
    out = torch.zeros((n, H * c), dtype=q.dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    positions = _i32([k - 1 for k in lengths])
    q2 = q.reshape(n, -1).contiguous()
    if how == "rows":
        kernels.latent_attention_rows(q2, out, cache, table, _i32(list(range(n))), positions, sink, H, c, r, page, 1.0, None, status)
    else:
        first, start = _i32(list(range(n + 1))), positions
        if how == "portions":
            kernels.latent_attention_mma(q2, out, cache, table, first, start, positions, sink, H, c, r, page, 1.0, None, status,
                                         max_rows_per_seq=1)
        else:
            splits = int(how[len("decode"):])
            part_o = torch.zeros((n, H * splits * c), device=DEV)
            part_ml = torch.zeros((n, H * splits * 2), device=DEV)
            kernels.latent_attention_mma(q2, out, cache, table, first, start, positions, sink, H, c, r, page, 1.0, None, status,
                                         decode=True, splits=splits, part_o=part_o, part_ml=part_ml)
    assert int(status.item()) == 0
    return out.float().cpu().numpy().reshape(n, H, c)


@pytest.mark.parametrize("how, dtype, H, c, r", [
    ("rows", torch.float32, 3, 16, 4), ("rows", torch.bfloat16, 3, 16, 4), ("rows", torch.bfloat16, 5, 64, 16),
    ("portions", torch.bfloat16, 3, 64, 16), ("portions", torch.bfloat16, 16, 128, 32), ("portions", torch.bfloat16, 20, 64, 64),
    ("decode1", torch.bfloat16, 3, 64, 16), ("decode3", torch.bfloat16, 16, 128, 32), ("decode7", torch.bfloat16, 20, 64, 32)])
def test_latent_attention_reads_the_right_keys(how, dtype, H, c, r):
    """Crafted cache rows: every key scores 0 except one, far back or at a page's or a tile's edge, that scores 12; the
    output must be that token's latent (less the sink's share). Pages are scattered; pages of nobody hold poison."""
    page, w, n_pages = 16, c + r, 64
    rng = np.random.default_rng(4)
    for length, hot in [(300, 0), (300, 15), (300, 16), (300, 63), (300, 64), (300, 255), (300, 299), (17, 16), (16, 15),
                        (1, 0), (257, 128), (65, 64), (64, 63)]:
        cache = torch.full((n_pages, 1, page, w), 50.0, dtype=dtype, device=DEV)            # poison
        order = rng.permutation(n_pages)[:-(-length // page)]
        latents = np.round(rng.standard_normal((length, c)) * 4) / 4                         # exact in bfloat16
        rows = np.zeros((length, w))
        rows[:, :c] = latents
        rows[hot, c:] = 1.0                                                                  # only the rotated part scores
        host = torch.full((n_pages, 1, page, w), 50.0, dtype=torch.float32)
        for t in range(length):
            host[order[t // page], 0, t % page] = torch.tensor(rows[t], dtype=torch.float32)
        cache.copy_(host.to(dtype))
        q = np.zeros((1, H, w))
        q[0, :, c] = 12.0                                                                     # scale 1: the hot key scores 12
        sink = np.resize(np.array([-30.0, 0.0, 12.0]), H)
        table = torch.full((1, 24), -1, dtype=torch.int32, device=DEV)
        table[0, :len(order)] = _i32(list(order))
        got = _run_latent_kernel(how, torch.tensor(q, dtype=dtype, device=DEV), cache, table, [length],
                                 torch.tensor(sink, dtype=torch.float32, device=DEV), H, c, r, page)[0]
        e = np.exp(12.0)
        others = latents.sum(0) - latents[hot]
        for head in range(H):
            want = (e * latents[hot] + others) / (e + (length - 1) + np.exp(sink[head]))
            np.testing.assert_allclose(got[head], want, atol=2e-2 if dtype == torch.bfloat16 else 1e-4,
                                       err_msg=f"{how}: length {length}, hot key {hot}, head {head}")


@pytest.mark.parametrize("H, c, r", [(6, 64, 16), (16, 128, 32), (24, 64, 32), (1, 128, 64)])
def test_latent_attention_tensor_core_kernel_equals_the_plain_one(H, c, r):
    """Random queries and caches, several requests of unequal lengths: the tensor-core kernel (portions of several rows;
    decoding with the keys in one, two and five shares) against softmax in float64."""
    from glassbox_b200 import kernels
    page, w, n_pages = 16, c + r, 96
    rng = np.random.default_rng(H)
    lengths, portions = [200, 37, 1, 130], [70, 37, 1, 5]              # tokens held, of which the last ones come now
    host = torch.tensor(rng.standard_normal((n_pages, 1, page, w)), dtype=torch.bfloat16)
    cache = host.to(DEV)
    free = list(rng.permutation(n_pages))
    table = torch.full((len(lengths), 16), -1, dtype=torch.int32)
    for s, n in enumerate(lengths):
        for i in range(-(-n // page)):
            table[s, i] = int(free.pop())
    sink = rng.standard_normal(H) * 2
    scale = 0.3 / np.sqrt(w)

    def reference(s, pos, qrow):                                        # qrow [H, w]
        keys = np.stack([host[table[s, t // page], 0, t % page].float().numpy() for t in range(pos + 1)]).astype(np.float64)
        sc = qrow @ keys.T * scale
        mx = np.maximum(sc.max(-1), sink)
        e = np.exp(sc - mx[:, None])
        return (e / (e.sum(-1) + np.exp(sink - mx))[:, None]) @ keys[:, :c]

    sink_t = torch.tensor(sink, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    # portions
    meta = _steps_meta([(n - k, k) for n, k in zip(lengths, portions)], [0] * len(lengths))
    q = torch.tensor(rng.standard_normal((meta["n"], H, w)), dtype=torch.bfloat16)
    out = torch.zeros((meta["n"], H * c), dtype=torch.bfloat16, device=DEV)
    kernels.latent_attention_mma(q.reshape(meta["n"], -1).to(DEV), out, cache, table.to(DEV), meta["first"], meta["start"],
                                 meta["positions"], sink_t, H, c, r, page, scale, None, status, max_rows_per_seq=max(portions))
    got = out.float().cpu().numpy().reshape(meta["n"], H, c)
    row = 0
    for s, (n, k) in enumerate(zip(lengths, portions)):
        for i in (0, 1, k // 2, k - 1):
            if i < k:
                want = reference(s, n - k + i, q[row + i].float().numpy().astype(np.float64))
                np.testing.assert_allclose(got[row + i], want, atol=0.03, err_msg=f"portion of request {s}, row {i}")
        row += k
    # decoding: each request's last token
    qd = torch.tensor(rng.standard_normal((len(lengths), H, w)), dtype=torch.bfloat16)
    for how in ("decode1", "decode2", "decode5"):
        got = _run_latent_kernel(how, qd.to(DEV), cache, table.to(DEV), lengths, sink_t * 0 + sink_t, H, c, r, page)
        # (the helper uses scale 1: fold the scale into the reference's queries instead)
        for s, n in enumerate(lengths):
            want = reference(s, n - 1, qd[s].float().numpy().astype(np.float64) / scale)
            np.testing.assert_allclose(got[s], want, atol=0.03, err_msg=f"{how}, request {s}")
    assert int(status.item()) == 0


# ------------------------------------------------------------------------------------------- whole models
_MODELS = {}


def _model(name, tmp_path_factory, seed=21, sharpen=1.0):
    key = (name, seed, sharpen)
    if key not in _MODELS:
        cfg = zu.CONFIGS[name]()
        tensors = zu.random_weights(cfg, seed, sharpen)
        folder = zu.write_model(str(tmp_path_factory.mktemp(f"zx_{name}_{seed}")), cfg, tensors)
        _MODELS[key] = (cfg, zu.as_float64(tensors), folder, {})
    return _MODELS[key]


def _want(model, tokens):
    cfg, W, _, memo = model
    key = tuple(tokens)
    if key not in memo:
        memo[key] = plain.forward(cfg, W, list(tokens))
    return memo[key]


def _tokens(cfg, n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], n)]


def _engine(folder, dtype, **kw):
    from glassbox_b200.engine.engine import Engine
    args = dict(cache_tokens=512, page_size=16, max_batch_tokens=256, max_requests=4)
    args.update(kw)
    return Engine(folder, dtype, **args)


@pytest.mark.parametrize("name, dtype", [(n, "float32") for n in sorted(zu.CONFIGS)] + [("odd", "bfloat16"), ("even", "bfloat16")])
def test_whole_prompt_and_token_by_token(name, dtype, tmp_path_factory):
    # ("ones" runs in float32 only: its norms run over eight numbers, and where such a vector happens to be small,
    # dividing by its size magnifies bfloat16 rounding until the comparison says nothing)
    model = _model(name, tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, dtype)
    for n, seed in [(1, 1), (2, 2), (45, 3)]:                      # the first tokens of a sequence; a page border and beyond
        toks = _tokens(cfg, n, seed)
        want = _want(model, toks)
        got = zu.run_schedule(eng, {"r": toks}, [[("r", n)]])["r"]
        assert_logits_close(got, want, dtype, f"{name} whole {n}")
        got = zu.run_schedule(eng, {"r": toks}, [[("r", 1)] for _ in range(n)])["r"]
        assert_logits_close(got, want, dtype, f"{name} token by token {n}")


def test_sizes_that_fit_no_vector_width_run_in_bfloat16_too(tmp_path_factory):
    """Odd row lengths in bfloat16: rows that start on two-byte boundaries only. The model is too small for a sharp
    comparison in bfloat16 (see above); what must hold is that every kernel takes the shapes, reads no neighbour's numbers
    (the logits stay near the plain ones) and that cutting the prompt changes nothing beyond rounding."""
    model = _model("ragged", tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, "bfloat16")
    toks = _tokens(cfg, 41, 5)
    want = _want(model, toks)
    whole = zu.run_schedule(eng, {"r": toks}, [[("r", 41)]])["r"]
    cut = zu.run_schedule(eng, {"r": toks}, [[("r", 17)], [("r", 2)], [("r", 21)], [("r", 1)]])["r"]
    assert np.isfinite(whole).all()
    assert np.abs(whole - want).mean() <= 0.05 * want.std()
    assert np.abs(whole - cut).mean() <= 0.02 * want.std()


@pytest.mark.parametrize("name", ["odd", "even"])
def test_portions_of_every_size(name, tmp_path_factory):
    model = _model(name, tmp_path_factory, sharpen=3.0)
    cfg, _, folder, _ = model
    eng = _engine(folder, "float32")
    toks = _tokens(cfg, 83, 7)
    want = _want(model, toks)
    for sizes in ([2] * 41 + [1], [3, 2, 16, 1, 15, 17, 2, 2, 25], [16, 16, 16, 16, 16, 3], [31, 2, 33, 17], [1, 82]):
        assert sum(sizes) == len(toks)
        got = zu.run_schedule(eng, {"r": toks}, [[("r", k)] for k in sizes])["r"]
        assert_logits_close(got, want, "float32", f"{name} portions {sizes[:4]}...")


@pytest.mark.parametrize("name, dtype", [("odd", "float32"), ("even", "float32"), ("even", "bfloat16")])
def test_mixed_batches_equal_each_request_alone(name, dtype, tmp_path_factory):
    """Unequal requests side by side, portions beside single tokens, requests that sit out a step, more requests than
    slots over time and a pool that only holds what is live: slots and pages are freed and used again."""
    model = _model(name, tmp_path_factory, sharpen=3.0 if dtype == "float32" else 1.0)
    cfg, _, folder, _ = model
    eng = _engine(folder, dtype, cache_tokens=192, max_requests=3)
    reqs = {"a": _tokens(cfg, 70, 11), "b": _tokens(cfg, 9, 12), "c": _tokens(cfg, 33, 13), "d": _tokens(cfg, 50, 14),
            "e": _tokens(cfg, 1, 15), "f": _tokens(cfg, 18, 16)}
    schedule = [[("a", 30), ("b", 2)], [("b", 1), ("a", 2), ("c", 16)], [("a", 1), ("b", 1), ("c", 1)],
                [("c", 16), ("b", 5)],                              # b and c end: their slots and pages go back
                [("a", 1)], [("d", 20), ("a", 2)], [("e", 1), ("d", 1), ("a", 1)], [("d", 29), ("a", 1)],
                [("f", 2), ("a", 1)], [("f", 16), ("a", 25)]] + [[("a", 1)]] * 6
    want = {k: _want(model, v) for k, v in reqs.items()}
    got = zu.run_schedule(eng, reqs, schedule)
    for k in reqs:
        assert_logits_close(got[k], want[k], dtype, f"{name} mixed, request {k}")
    eng.cache.check_invariants()
    assert len(eng.cache.free_slots) == eng.cache.max_requests


def test_long_decoding_through_recorded_steps(tmp_path_factory):
    model = _model("even", tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, "float32")
    a, b = _tokens(cfg, 150, 31), _tokens(cfg, 140, 32)
    schedule = [[("a", 20)], [("b", 3)]] + [[("a", 1), ("b", 1)]] * 130 + [[("b", 7)]]
    got = zu.run_schedule(eng, {"a": a, "b": b}, schedule)
    assert eng.graph_replays > 100                                   # the decode steps ran as recorded graphs
    assert_logits_close(got["a"], _want(model, a), "float32", "long decoding a")
    assert_logits_close(got["b"], _want(model, b), "float32", "long decoding b")


def test_a_slot_that_is_used_again_starts_from_zero(tmp_path_factory):
    model = _model("odd", tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, "float32", max_requests=1, cache_tokens=64)
    for seed in (41, 42, 43):
        toks = _tokens(cfg, 40, seed)
        got = zu.run_schedule(eng, {"r": toks}, [[("r", 25)], [("r", 15)]])["r"]
        assert_logits_close(got, _want(model, toks), "float32", f"slot reuse {seed}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(dtype, tmp_path_factory):
    import glassbox_b200
    model = _model("even", tmp_path_factory, seed=5)
    cfg, W, folder, _ = model
    llm = glassbox_b200.load(folder, dtype, blocks=64, budget=32, max_seqs=3, prefix_cache=True)
    prompts = [_tokens(cfg, 37, 51), _tokens(cfg, 5, 52), _tokens(cfg, 70, 53), _tokens(cfg, 1, 54)]
    outs = llm.generate(prompts, max_tokens=12)
    for p, out in zip(prompts, outs):
        seq = list(p)
        for i, tok in enumerate(out):
            logits = plain.forward(cfg, W, seq)[-1]
            best = int(np.argmax(logits))
            if dtype == "bfloat16" and tok != best:
                top2 = np.sort(logits)[-2:]
                assert logits[tok] >= top2[1] - 0.08 * logits.std(), f"token {i}: {tok} is not near the best"
                break                                                # rounding chose the runner-up: the texts part ways
            assert tok == best, f"{dtype} prompt of {len(p)}: token {i} is {tok}, plain says {best}"
            seq.append(tok)
