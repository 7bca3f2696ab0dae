"""Lonorax on the GPU against the plain float64 implementation (``tests/plain/lonorax_plain.py``): each mechanism's
kernel alone, then whole models under every way of cutting and batching their requests, through the engine's own step
function, cache manager, scheduler and entry point. Sizes are the tests' own (``lonorax_util.CONFIGS``)."""
import numpy as np
import pytest
import torch

import conftest
from plain import lonorax_plain as plain
import lonorax_util as lu
import zurerax_util as zu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# bfloat16 against float64: a handful of roundings per branch (norm out, three products, activations), summed through the
# streams over four layers. A mixture of experts adds something a dense model does not have: where two experts' choice
# scores lie closer than the rounding of the router's input, bfloat16 picks the other one, and that token's logits (and,
# through the recurrent state and the keys, faintly the tokens after it) differ by a discrete amount. So the bound holds
# for nine rows in ten and for the median row, not for every row. Faults in which key, state or expert a bfloat16 kernel
# reads are caught by the crafted tests below and by the float32 runs of the same code, which are held to 1e-4.
BF16_REL_MAX, BF16_REL_MEAN, BF16_ROWS_OFF = 0.25, 0.02, 0.1


def assert_logits_close(got, want, dtype, what=""):
    if dtype == "float32":
        return conftest.assert_logits_close(got, want, dtype, what)
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert np.isfinite(got).all(), f"{what}: not finite"
    diff, spread = np.abs(got - want), want.std()
    off = diff.max(1) > BF16_REL_MAX * spread
    assert off.sum() <= max(1, BF16_ROWS_OFF * len(off)), \
        f"{what}: {int(off.sum())} of {len(off)} rows differ by more than {BF16_REL_MAX} x spread {spread:.3e} (worst {diff.max():.3e})"
    assert np.median(diff.mean(1)) <= BF16_REL_MEAN * spread, \
        f"{what}: the median row's mean abs diff {np.median(diff.mean(1)):.3e} > {BF16_REL_MEAN} x spread {spread:.3e}"


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def _f32(a):
    return torch.tensor(np.asarray(a, dtype=np.float32), device=DEV)


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
@pytest.mark.parametrize("S, d", [(1, 48), (3, 56), (4, 128), (8, 33)])
def test_streams_fold_read_norm_and_gather(S, d):
    from glassbox_b200 import kernels
    rng = np.random.default_rng(S * 100 + d)
    n, eps = 9, 1e-5
    xs = rng.standard_normal((n, S, d)) * 3 + 1.0
    y = rng.standard_normal((n, d))
    mix, write, read = rng.standard_normal((S, S)), rng.standard_normal(S), rng.standard_normal(S)
    w, b = rng.standard_normal(d), rng.standard_normal(d)
    positions = _i32([0, 1, 2, -1, 5, 6, 7, 8, 9])                       # row 3 is a padding row: left alone
    # plain: the streams as [S, n, d]
    new = plain.stream_write(xs.transpose(1, 0, 2), mix, write, y)
    want_h = plain.layer_norm(plain.stream_read(new, read), w, b, eps)
    dev = _f32(xs.reshape(n, S * d))
    h = torch.zeros((n, d), dtype=torch.float32, device=DEV)
    kernels.streams_step(dev, S, fold=(_f32(y), _f32(mix), _f32(write)), read=_f32(read), norm=(_f32(w), _f32(b), eps), h=h,
                         positions=positions)
    live = [0, 1, 2, 4, 5, 6, 7, 8]
    np.testing.assert_allclose(h.cpu().numpy()[live], want_h[live], atol=2e-5, rtol=1e-5)
    got_xs = dev.cpu().numpy().reshape(n, S, d)
    np.testing.assert_allclose(got_xs[live], new.transpose(1, 0, 2)[live], atol=1e-5, rtol=1e-5)
    np.testing.assert_array_equal(got_xs[3], xs[3].astype(np.float32))
    assert float(h[3].abs().max()) == 0.0
    # the same fold with y handed over as its parts: a weighted sum of rows plus a gated shared row
    top = 3
    pair, pw, gate = rng.standard_normal((n, top, d)), rng.uniform(0.2, 1.5, (n, top)), rng.uniform(0, 1, n)
    shared = y - np.einsum("nk,nkd->nd", pw, pair)
    shared /= gate[:, None]
    for parts in (kernels.WeightedRows(_f32(pair.reshape(n, top * d)), _f32(pw), _f32(shared), _f32(gate)),
                  kernels.WeightedRows(_f32(pair.reshape(n, top * d)), _f32(pw), _f32(shared * gate[:, None]), None)):
        dev3 = _f32(xs.reshape(n, S * d))
        h3 = torch.zeros((n, d), dtype=torch.float32, device=DEV)
        kernels.streams_step(dev3, S, fold=(parts, _f32(mix), _f32(write)), read=_f32(read), norm=(_f32(w), _f32(b), eps), h=h3,
                             positions=positions)
        np.testing.assert_allclose(h3.cpu().numpy()[live], want_h[live], atol=2e-4, rtol=1e-4)
        np.testing.assert_allclose(dev3.cpu().numpy().reshape(n, S, d)[live], new.transpose(1, 0, 2)[live], atol=1e-4, rtol=1e-4)
    # the end of the streams: gathered rows, the plain sum, a fold that is computed but not stored
    dev2 = _f32(xs.reshape(n, S * d))
    rows = _i32([7, 0, 0, 4])
    hs = torch.zeros((4, d), dtype=torch.bfloat16, device=DEV)
    total = torch.zeros((4, d), dtype=torch.float32, device=DEV)
    kernels.streams_step(dev2, S, fold=(_f32(y), _f32(mix), _f32(write)), norm=(_f32(w), None, eps), h=hs, u_out=total, rows=rows)
    np.testing.assert_array_equal(dev2.cpu().numpy(), xs.reshape(n, S * d).astype(np.float32))
    np.testing.assert_allclose(total.cpu().numpy(), new.sum(0)[[7, 0, 0, 4]], atol=2e-5, rtol=1e-5)
    np.testing.assert_allclose(hs.float().cpu().numpy(), plain.layer_norm(new.sum(0), w, 0.0, eps)[[7, 0, 0, 4]], atol=0.03, rtol=0.01)
    # one stream and nothing to fold: the plain layer norm
    if S == 1:
        out = torch.zeros((n, d), dtype=torch.float32, device=DEV)
        kernels.streams_step(_f32(xs.reshape(n, d)), 1, norm=(_f32(w), _f32(b), eps), h=out)
        np.testing.assert_allclose(out.cpu().numpy(), plain.layer_norm(xs.reshape(n, d), w, b, eps), atol=2e-5, rtol=1e-5)
    bc = torch.zeros((n, S * d), dtype=torch.float32, device=DEV)
    kernels.streams_broadcast(_f32(y), bc, S)
    np.testing.assert_array_equal(bc.cpu().numpy().reshape(n, S, d), np.repeat(y.astype(np.float32)[:, None], S, 1))


class _PagedRequests:
    """A paged cache for a few requests whose pages lie scattered and interleaved in the pool."""

    def __init__(self, lengths, G, D, V, page, dtype, seed=0):
        rng = np.random.default_rng(seed)
        self.page, self.G = page, G
        need = [-(-n // page) for n in lengths]
        order = rng.permutation(sum(need) + 3)
        self.tables, at = [], 0
        for k in need:
            self.tables.append([int(p) for p in order[at:at + k]])
            at += k
        self.pages = sum(need) + 3
        self.width = max(need)
        self.k = torch.zeros((self.pages, G, page, D), dtype=dtype, device=DEV)
        self.v = torch.zeros((self.pages, G, page, V), dtype=dtype, device=DEV)

    def table(self, seqs):
        return _i32([self.tables[s] + [-1] * (self.width - len(self.tables[s])) for s in seqs])

    def slots(self, rows):
        """rows: [(request, position)] -> slot of each row."""
        return _i32([self.tables[s][p // self.page] * self.page + p % self.page for s, p in rows])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, G, D, V, rot, window, page", [(6, 2, 20, 12, 8, 7, 16), (4, 1, 64, 64, 32, 33, 16), (3, 3, 10, 7, 10, None, 8),
                                                          (2, 1, 128, 32, 0, 17, 16)])
def test_sigmoid_attention_kernels(dtype, H, G, D, V, rot, window, page):
    """Norm, rotation and cache write, then attention, for two requests in portions (the cache carries the earlier
    tokens), against the plain implementation over the whole sequences."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(H * 1000 + D)
    lengths, eps, scale, base = [45, 23], 1e-5, D ** -0.5, 700.0
    qkv = [rng.standard_normal((n, (H + G) * D + G * V)) for n in lengths]
    gq, gk, pb = 1 + 0.3 * rng.standard_normal(D), 1 + 0.3 * rng.standard_normal(D), rng.standard_normal(H) - 1.0
    want = []
    for r, n in enumerate(lengths):
        # the plain mixer with identity projections: h = the stacked row itself
        m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": scale}
        if window:
            m["mask"] = {"size": window}
        if rot:
            m["rot"] = {"dims": rot, "base": base}
        cols = qkv[r].shape[1]
        eye = np.eye(cols)
        W = {"q": eye[:H * D], "k": eye[H * D:(H + G) * D], "v": eye[(H + G) * D:], "q.norm": gq, "k.norm": gk, "pb": pb,
             "o": np.eye(H * V)}
        want.append(plain.sigmoid_attention(qkv[r], W, "", m, eps))
    cache = _PagedRequests(lengths, G, D, V, page, dtype, seed=D)
    inv = _f32(base ** (-2.0 * np.arange(rot // 2) / rot)) if rot else None
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = [np.zeros((n, H * V)) for n in lengths]
    at = [0, 0]
    for step in ([(0, 17), (1, 2)], [(1, 1), (0, 1)], [(0, 27), (1, 20)]):        # portions beside single tokens, cut mid-page
        rows = [(r, at[r] + i) for r, k in step for i in range(k)]
        x = _f32(np.concatenate([qkv[r][at[r]:at[r] + k] for r, k in step]))
        n = len(rows)
        q = torch.zeros((n, H * D), dtype=dtype, device=DEV)
        out = torch.zeros((n, H * V), dtype=dtype, device=DEV)
        positions, row_seq = _i32([p for _, p in rows]), _i32([i for i, (r, k) in enumerate(step) for _ in range(k)])
        kernels.qk_norm_rope_write(x, _f32(gq), _f32(gk), inv, positions, cache.slots(rows), q, cache.k, cache.v, H, G, D, V, rot, eps,
                                   page, True, status)
        single = all(k == 1 for _, k in step) and kernels.sigmoid_attention_decode_supported(dtype, V)   # the kernel that decoding uses
        attend = kernels.sigmoid_attention_decode if single else kernels.sigmoid_attention_rows
        attend(q, out, cache.k, cache.v, cache.table([r for r, _ in step]), row_seq, positions, _f32(pb), H, G, D, V, page, scale, window,
               status)
        o = out.float().cpu().numpy()
        i = 0
        for r, k in step:
            got[r][at[r]:at[r] + k] = o[i:i + k]
            i += k
            at[r] += k
    assert int(status.item()) == 0
    for r in range(2):
        if dtype == torch.float32:
            np.testing.assert_allclose(got[r], want[r], atol=3e-5, rtol=1e-5)
        else:
            assert np.abs(got[r] - want[r]).max() <= 0.03 * max(1.0, np.abs(want[r]).max())


@pytest.mark.parametrize("H, G, D, V, rot, window, page", [(4, 2, 64, 64, 32, 33, 16), (2, 1, 128, 32, 64, 100, 16), (3, 3, 32, 128, 0, None, 8),
                                                          (8, 2, 128, 128, 32, 64, 32)])
def test_sigmoid_attention_on_the_tensor_cores(H, G, D, V, rot, window, page):
    """Prompt portions through the tile kernel: three requests of unequal length, the second and third continuing from a
    cache that earlier portions filled, one padding sequence; against the plain implementation over whole sequences."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(H * 1000 + D + V)
    lengths, eps, scale, base, dtype = [150, 70, 3], 1e-5, D ** -0.5, 700.0, torch.bfloat16
    qkv = [rng.standard_normal((n, (H + G) * D + G * V)) for n in lengths]
    gq, gk, pb = 1 + 0.3 * rng.standard_normal(D), 1 + 0.3 * rng.standard_normal(D), rng.standard_normal(H) - 2.0
    want = []
    for r, n in enumerate(lengths):
        m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": scale}
        if window:
            m["mask"] = {"size": window}
        if rot:
            m["rot"] = {"dims": rot, "base": base}
        eye = np.eye(qkv[r].shape[1])
        W = {"q": eye[:H * D], "k": eye[H * D:(H + G) * D], "v": eye[(H + G) * D:], "q.norm": gq, "k.norm": gk, "pb": pb, "o": np.eye(H * V)}
        want.append(plain.sigmoid_attention(qkv[r], W, "", m, eps))
    cache = _PagedRequests(lengths, G, D, V, page, dtype, seed=V)
    inv = _f32(base ** (-2.0 * np.arange(rot // 2) / rot)) if rot else None
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = [np.zeros((n, H * V)) for n in lengths]
    at = [0, 0, 0]
    for step in ([(1, 37), None, (0, 150)], [(2, 2), (1, 33)], [(2, 1)]):
        live = [e for e in step if e is not None]
        rows = [(r, at[r] + i) for r, k in live for i in range(k)]
        meta = _steps_meta([None if e is None else (at[e[0]], e[1]) for e in step], [0] * len(step))
        x = np.zeros((meta["n"], qkv[0].shape[1]))
        slots, row = [-1] * meta["n"], 0
        for e in step:
            if e is None:
                row += 1
                continue
            x[row:row + e[1]] = qkv[e[0]][at[e[0]]:at[e[0]] + e[1]]
            for i in range(e[1]):
                p = at[e[0]] + i
                slots[row + i] = cache.tables[e[0]][p // page] * page + p % page
            row += e[1]
        n = meta["n"]
        q = torch.zeros((n, H * D), dtype=dtype, device=DEV)
        out = torch.zeros((n, H * V), dtype=dtype, device=DEV)
        kernels.qk_norm_rope_write(_f32(x), _f32(gq), _f32(gk), inv, meta["positions"], _i32(slots), q, cache.k, cache.v, H, G, D, V, rot,
                                   eps, page, True, status)
        tables = _i32([[-1] * cache.width if e is None else cache.tables[e[0]] + [-1] * (cache.width - len(cache.tables[e[0]])) for e in step])
        kernels.sigmoid_attention_tiles(q, out, cache.k, cache.v, tables, meta["first"], meta["start"], max(e[1] for e in live),
                                        _f32(pb), H, G, D, V, page, scale, window, status)
        o, row = out.float().cpu().numpy(), 0
        for e in step:
            if e is None:
                row += 1
                continue
            got[e[0]][at[e[0]]:at[e[0]] + e[1]] = o[row:row + e[1]]
            row += e[1]
            at[e[0]] += e[1]
    assert int(status.item()) == 0
    for r in range(3):
        assert np.abs(got[r] - want[r]).max() <= 0.03 * max(1.0, np.abs(want[r]).max()), f"request {r}"


@pytest.mark.parametrize("window, page", [(5, 16), (64, 16), (65, 16), (100, 8), (None, 16)])
def test_which_keys_a_tile_of_rows_sees(window, page):
    """The crafted cache of the test below through the tile kernel: one portion of 200 rows that starts at position 130 (its
    tiles begin in the middle of a page and of a window), then the exact sums say which keys every row took."""
    from glassbox_b200 import kernels
    D, V, T, start, dtype = 32, 64, 330, 130, torch.bfloat16
    cache = _PagedRequests([T], 1, D, V, page, dtype, seed=3)
    for j in range(T):
        pg, off = cache.tables[0][j // page], j % page
        cache.k[pg, 0, off, 0] = 8.0
        cache.v[pg, 0, off, j // 8] = 2.0 ** (j % 8)
    n = T - start
    q = torch.zeros((n, D), dtype=dtype, device=DEV); q[:, 0] = 8.0
    out = torch.zeros((n, V), dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.sigmoid_attention_tiles(q, out, cache.k, cache.v, cache.table([0]), _i32([0, n]), _i32([start]), n, None, 1, 1, D, V, page,
                                    1.0, window, status)
    assert int(status.item()) == 0
    got = out.float().cpu().numpy()
    for i in range(n):
        want = np.zeros(V)
        for j in range(T):
            if plain.visible(start + i, j, window):
                want[j // 8] += 2.0 ** (j % 8)
        np.testing.assert_array_equal(got[i], want, err_msg=f"position {start + i}, window {window}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_many_single_tokens_share_a_groups_keys(dtype):
    """With many rows the decode kernel takes the four query heads of a key/value group through one block. 80 requests of
    unequal length, one token each: every row against the plain sum over its own keys."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(9)
    H, G, D, V, page, window, n = 8, 2, 32, 64, 16, 37, 80
    lengths = [int(x) for x in rng.integers(1, 120, n)]
    cache = _PagedRequests(lengths, G, D, V, page, dtype, seed=1)
    cache.k.copy_(torch.randn(cache.k.shape, device=DEV))
    cache.v.copy_(torch.randn(cache.v.shape, device=DEV))
    q = torch.randn((n, H * D), device=DEV).to(dtype)
    pb = rng.standard_normal(H) - 1.0
    out = torch.zeros((n, H * V), dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    positions = [L - 1 for L in lengths]
    kernels.sigmoid_attention_decode(q, out, cache.k, cache.v, cache.table(list(range(n))), _i32(list(range(n))), _i32(positions), _f32(pb),
                                     H, G, D, V, page, 0.3, window, status)
    assert int(status.item()) == 0
    got = out.float().cpu().numpy().reshape(n, H, V)
    k64, v64, q64 = cache.k.float().cpu().numpy().astype(np.float64), cache.v.float().cpu().numpy().astype(np.float64), \
        q.float().cpu().numpy().astype(np.float64).reshape(n, H, D)
    for r in range(n):
        want = np.zeros((H, V))
        for j in range(lengths[r]):
            if plain.visible(positions[r], j, window):
                pg, off = cache.tables[r][j // page], j % page
                for h in range(H):
                    want[h] += plain.logistic(q64[r, h] @ k64[pg, h // (H // G), off] * 0.3 + pb[h]) * v64[pg, h // (H // G), off]
        tol = 1e-4 if dtype == torch.float32 else 0.03
        assert np.abs(got[r] - want).max() <= tol * max(1.0, np.abs(want).max()), f"row {r}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window, page", [(5, 16), (16, 16), (17, 16), (40, 8), (None, 16)])
def test_which_keys_a_row_sees(dtype, window, page):
    """Crafted cache: every key has the same direction as every query, so that every visible key weighs sigmoid(large) = 1
    exactly, and the value of key j is 2^(j mod 8) in channel j / 8: the output then spells out, bit by bit, which keys were
    summed. Rows at page borders, at the first positions, just inside and just outside the window, 300 keys back."""
    from glassbox_b200 import kernels
    D, V, T = 16, 64, 330
    cache = _PagedRequests([T], 1, D, V, page, dtype, seed=3)
    k = np.zeros((T, D)); k[:, 0] = 8.0
    v = np.zeros((T, V))
    for j in range(T):
        v[j, j // 8] = 2.0 ** (j % 8)
    for j in range(T):
        pg, off = cache.tables[0][j // page], j % page
        cache.k[pg, 0, off] = torch.tensor(k[j], dtype=dtype)
        cache.v[pg, 0, off] = torch.tensor(v[j], dtype=dtype)
    rows = [0, 1, 2, 7, 8, 15, 16, 17, 31, 32, 39, 40, 41, 47, 48, 63, 64, 65, 300, 319, 320, 329]
    q = torch.zeros((len(rows), D), dtype=dtype, device=DEV); q[:, 0] = 8.0
    out = torch.zeros((len(rows), V), dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for attend in (kernels.sigmoid_attention_rows, kernels.sigmoid_attention_decode):
        out.zero_()
        attend(q, out, cache.k, cache.v, cache.table([0]), _i32([0] * len(rows)), _i32(rows), None, 1, 1, D, V, page, 1.0, window, status)
        assert int(status.item()) == 0
        got = out.float().cpu().numpy()
        for i, p in enumerate(rows):
            want = np.zeros(V)
            for j in range(T):
                if plain.visible(p, j, window):
                    want[j // 8] += 2.0 ** (j % 8)
            np.testing.assert_array_equal(got[i], want, err_msg=f"{attend.__name__}: position {p}, window {window}")


@pytest.mark.parametrize("width", [1, 13, 72, 256])
@pytest.mark.parametrize("bound", [0, 600])
def test_mingru_scan_carries_its_state(width, bound):
    """Portions of 1, 2, a few and many rows (the kernel cuts long ones into pieces), requests side by side with a padding
    sequence between them, slots of other requests untouched."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(width)
    lens = {"a": 150, "b": 37}
    proj = {k: rng.standard_normal((n, 3 * width)) * 2 for k, n in lens.items()}
    bz, bx = rng.standard_normal(width), rng.standard_normal(width)
    W = {"z": np.eye(3 * width)[:width], "x": np.eye(3 * width)[width:2 * width], "g": np.eye(3 * width)[2 * width:], "z.b": bz,
         "x.b": bx, "o": np.eye(width)}
    want = {k: plain.mingru(proj[k], W, "") for k in lens}
    state = torch.full((4, width + 3), 7.0, dtype=torch.float32, device=DEV)
    slot = {"a": 2, "b": 0}
    state[2, 1:1 + width] = 0.0
    state[0, 1:1 + width] = 0.0
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = {k: np.zeros((n, width)) for k, n in lens.items()}
    at = {"a": 0, "b": 0}
    for step in ([("a", 1), None, ("b", 2)], [("b", 1), ("a", 1)], [("a", 2), ("b", 30)], [("a", 129), None], [("b", 4), ("a", 17)]):
        meta = _steps_meta([None if e is None else (at[e[0]], e[1]) for e in step], [-1 if e is None else slot[e[0]] for e in step])
        x = np.zeros((meta["n"], 3 * width))
        row = 0
        for e in step:
            if e is None:
                row += 1
                continue
            x[row:row + e[1]] = proj[e[0]][at[e[0]]:at[e[0]] + e[1]]
            row += e[1]
        out = torch.zeros((meta["n"], width), dtype=torch.float32, device=DEV)
        kernels.mingru_scan(_f32(x), _f32(bz), _f32(bx), state, 1, out, meta["first"], meta["start"], meta["slots"], width, True, status,
                            max_rows=bound)          # (600: the form for long portions, 16 channels and 64 pieces per block)
        o, row = out.cpu().numpy(), 0
        for e in step:
            if e is None:
                row += 1
                continue
            got[e[0]][at[e[0]]:at[e[0]] + e[1]] = o[row:row + e[1]]
            row += e[1]
            at[e[0]] += e[1]
    assert int(status.item()) == 0
    for k in lens:
        np.testing.assert_allclose(got[k], want[k][0], atol=3e-5, rtol=2e-5)
        np.testing.assert_allclose(state[slot[k], 1:1 + width].cpu().numpy(), want[k][1], atol=2e-5, rtol=2e-5)
    assert float((state[1] - 7.0).abs().max()) == 0.0 and float((state[3] - 7.0).abs().max()) == 0.0
    assert float((state[:, 0] - 7.0).abs().max()) == 0.0 and float((state[:, 1 + width:] - 7.0).abs().max()) == 0.0


def _route_plain(h, Wr, corr, router):
    return [plain.route(h[t], {"router": Wr, "correction": corr}, "", router) for t in range(h.shape[0])]


@pytest.mark.parametrize("E, top, groups, d", [(6, 2, (3, 2), 56), (16, 4, (4, 3), 128), (5, 1, None, 33), (4, 1, (4, 2), 32), (8, 8, None, 40),
                                              (64, 6, (8, 3), 96)])
@pytest.mark.parametrize("n", [50, 300])                      # (300: the form that takes eight rows per block)
def test_router_choice_and_weights(E, top, groups, d, n):
    from glassbox_b200 import kernels
    rng = np.random.default_rng(E * 10 + top)
    h = rng.standard_normal((n, d))
    Wr, corr, wg = rng.standard_normal((E, d)) * 2 / np.sqrt(d), rng.standard_normal(E) * 0.5 - 0.7, rng.standard_normal(d) / np.sqrt(d)
    router = {"experts": E, "top": top, "scale": 1.7}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    want = _route_plain(h, Wr, corr, router)
    choice = torch.zeros((n, top), dtype=torch.int32, device=DEV)
    weight = torch.zeros((n, top), dtype=torch.float32, device=DEV)
    gate = torch.zeros((n, 1), dtype=torch.float32, device=DEV)
    positions = _i32(list(range(n)))
    g = groups or (1, 1)
    kernels.moe_route(_f32(h), _f32(Wr), _f32(corr), _f32(wg), positions, top, g[0], g[1], 1.7, choice, weight, gate)
    c, w = choice.cpu().numpy(), weight.cpu().numpy()
    for t in range(n):
        assert list(c[t]) == want[t][0], f"row {t}: chose {list(c[t])}, plain says {want[t][0]}"
        np.testing.assert_allclose(w[t], want[t][1], atol=1e-5, rtol=1e-5)
    np.testing.assert_allclose(gate.cpu().numpy()[:, 0], plain.logistic(h @ wg), atol=1e-5)


def test_router_on_crafted_scores():
    """Scores made by hand (the router matrix picks single channels of h), so that the rules that random numbers rarely
    separate decide the outcome: a group wins by the sum of its two best, not by its single best; a left-out group's
    experts lose even to negative choice scores; the correction moves the choice but not the weight."""
    from glassbox_b200 import kernels
    E, d = 6, 8
    logit = lambda s: float(np.log(s / (1 - s)))
    Wr = np.eye(E, d)
    # groups of two: {0,1}, {2,3}, {4,5}; keep 2 groups, take 3 experts
    scores = np.array([[0.9, 0.1, 0.6, 0.6, 0.5, 0.55],      # best single expert in group 0 (sum 1.0), groups 1 (1.2) and 2 (1.05) win
                       [0.5, 0.5, 0.5, 0.5, 0.5, 0.5]])
    corr = np.array([[0.0] * 6, [-0.9, -0.8, 0.2, -0.95, -0.7, 0.1]])
    expect = [[2, 3, 5], None]
    for t in range(2):
        h = np.zeros((1, d)); h[0, :E] = [logit(s) for s in scores[t]]
        want = plain.route(h[0], {"router": Wr, "correction": corr[t]}, "", {"experts": E, "top": 3, "scale": 2.0, "groups": {"count": 3, "keep": 2}})
        if expect[t] is not None:
            assert want[0] == expect[t]
        choice = torch.zeros((1, 3), dtype=torch.int32, device=DEV)
        weight = torch.zeros((1, 3), dtype=torch.float32, device=DEV)
        kernels.moe_route(_f32(h), _f32(Wr), _f32(corr[t]), None, _i32([0]), 3, 3, 2, 2.0, choice, weight, None)
        assert list(choice.cpu().numpy()[0]) == want[0]
        np.testing.assert_allclose(weight.cpu().numpy()[0], want[1], atol=1e-5)
    # second row: choice scores -0.4, -0.3 | 0.7, -0.45 | -0.2, 0.6: groups 1 (0.25) and 2 (0.4) are kept; the third expert
    # is 4 (-0.2), not 1 (-0.3, left out) and not 3 (-0.45); every weight is 0.5 * 2, whatever the correction
    assert want[0] == [2, 5, 4] and np.allclose(want[1], 1.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E, top, ff, d, shared", [(6, 2, 24, 56, 40), (4, 3, 11, 50, 0), (8, 2, 64, 128, 128)])
def test_experts_and_their_sum(dtype, E, top, ff, d, shared):
    from glassbox_b200 import kernels
    rng = np.random.default_rng(E + ff)
    n = 21
    rnd = lambda *s: torch.tensor(rng.standard_normal(s), dtype=torch.float32).to(dtype)
    h = rnd(n, d)
    up, down = rnd(E * ff, d) / np.sqrt(d), rnd(E * d, ff) / np.sqrt(ff)
    choice = np.stack([rng.permutation(E)[:top] for _ in range(n)]).astype(np.int32)
    weight = rng.uniform(0.1, 2.0, (n, top))
    positions = list(range(n)); positions[5] = -1
    pair = torch.zeros((n, top * d), dtype=torch.float32, device=DEV)
    kernels.moe_expert_rows(h.to(DEV), up.to(DEV), down.to(DEV), E, _i32(choice), _i32(positions), pair)
    h64, up64, down64 = (t.float().numpy().astype(np.float64) for t in (h, up, down))
    want = np.zeros((n, d))
    for t in range(n):
        for k in range(top):
            e = choice[t, k]
            want[t] += weight[t, k] * plain.expert(h64[t], up64[e * ff:(e + 1) * ff], down64[e * d:(e + 1) * d])
    sh = rng.standard_normal((n, d)) if shared else None
    gate = rng.uniform(0, 1, n) if shared else None
    if shared:
        want += gate[:, None] * sh
    out = torch.full((n, d), 2.0, dtype=torch.float32, device=DEV)
    kernels.moe_combine(pair, _f32(weight), _f32(sh) if shared else None, _f32(gate) if shared else None, _i32(positions), out, True)
    got = out.cpu().numpy()
    live = [t for t in range(n) if t != 5]
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    np.testing.assert_allclose(got[live], want[live] + 2.0, atol=tol * max(1.0, np.abs(want).max()), rtol=tol)
    assert np.all(got[5] == 2.0)                                             # a padding row is left alone
    kernels.moe_combine(pair, _f32(weight), None, None, _i32(positions), out, False)
    assert np.all(out.cpu().numpy()[5] == 2.0)


@pytest.mark.parametrize("E, top, ff, d, n", [(8, 2, 64, 128, 300), (16, 4, 40, 72, 77), (3, 3, 136, 64, 129)])
def test_grouped_experts_equal_the_row_form(E, top, ff, d, n):
    """The pairs sorted by expert and run as grouped tensor-core products, against the plain experts; some experts get no
    row, some more than a tile of 64, padding rows are skipped; the split row form (float32 activations) beside it."""
    from glassbox_b200 import kernels
    rng = np.random.default_rng(E + ff + n)
    rnd = lambda *s: torch.tensor(rng.standard_normal(s), dtype=torch.float32).bfloat16()
    h, up, down = rnd(n, d), rnd(E * ff, d) / np.sqrt(d), rnd(E * d, ff) / np.sqrt(ff)
    usable = [e for e in range(E) if e != 1 or E <= top]                         # expert 1 gets no row
    choice = np.stack([rng.permutation(usable)[:top] for _ in range(n)]).astype(np.int32)
    positions = list(range(n)); positions[7] = -1
    tables = torch.zeros(2 * (E + 1) + n * top, dtype=torch.int32, device=DEV)
    act = torch.zeros((n, top * ff), dtype=torch.bfloat16, device=DEV)
    pair = torch.full((n, top * d), 9.0, dtype=torch.float32, device=DEV)
    kernels.moe_experts_grouped(h.to(DEV), up.to(DEV), down.to(DEV), E, _i32(choice), _i32(positions), tables, act, pair)
    act32 = torch.zeros((n, top * ff), dtype=torch.float32, device=DEV)
    pair2 = torch.full((n, top * d), 9.0, dtype=torch.float32, device=DEV)
    kernels.moe_expert_halves(h.to(DEV), up.to(DEV), down.to(DEV), E, _i32(choice), _i32(positions), act32, pair2)
    h64, up64, down64 = (t.float().numpy().astype(np.float64) for t in (h, up, down))
    got, got2 = pair.cpu().numpy().reshape(n, top, d), pair2.cpu().numpy().reshape(n, top, d)
    for t in range(n):
        if t == 7:
            assert np.all(got[t] == 9.0) and np.all(got2[t] == 9.0)
            continue
        for k in range(top):
            e = choice[t, k]
            want = plain.expert(h64[t], up64[e * ff:(e + 1) * ff], down64[e * d:(e + 1) * d])
            np.testing.assert_allclose(got2[t, k], want, atol=2e-3 * max(1.0, np.abs(want).max()), rtol=2e-3)
            np.testing.assert_allclose(got[t, k], want, atol=2e-2 * max(1.0, np.abs(want).max()), rtol=2e-2)
    counts = tables[:E + 1].cpu().numpy()
    assert counts[E] == (n - 1) * top and (E <= top or counts[2] == counts[1])   # every live pair sorted; expert 1 empty


# ------------------------------------------------------------------------------------------- whole models
_MODELS = {}


def _model(name, tmp_path_factory, seed=1):
    key = (name, seed)
    if key not in _MODELS:
        cfg = lu.CONFIGS[name]()
        tensors = lu.random_weights(cfg, seed)
        folder = lu.write_model(str(tmp_path_factory.mktemp(f"lonorax_{name}")), cfg, tensors)
        _MODELS[key] = (cfg, lu.as_float64(tensors), folder, {})
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


def test_every_layer_against_the_plain_one(tmp_path_factory):
    """The residual after every layer (the sum of the streams), in float32: a fault shows in the layer that has it."""
    from glassbox_b200 import kernels
    from glassbox_b200.engine.engine import StepEntry
    from glassbox_b200.parts.block import HyperConnectionBlock
    model = _model("odd", tmp_path_factory)
    cfg, W, folder, _ = model
    toks = _tokens(cfg, 29, 3)
    want = []
    plain.forward(cfg, W, toks, per_layer=want)
    eng = _engine(folder, "float32", use_graphs=False)
    seen = []
    inner = HyperConnectionBlock.forward

    def spying(self, ctx, xs, cache, writes_cache, after_mixer=None):
        inner(self, ctx, xs, cache, writes_cache, after_mixer)
        total = torch.zeros((xs.shape[0], self.hidden_size), dtype=torch.float32, device=xs.device)
        kernels.streams_step(xs, self.streams, fold=ctx.pending_fold, u_out=total,
                             rows=torch.arange(xs.shape[0], dtype=torch.int32, device=xs.device))
        seen.append(total.cpu().numpy())

    HyperConnectionBlock.forward = spying
    try:
        eng.add_request("r", [])
        eng.step([StepEntry("r", toks, [0])])
    finally:
        HyperConnectionBlock.forward = inner
    assert len(seen) == len(want)
    for i, (g, w) in enumerate(zip(seen, want)):
        np.testing.assert_allclose(g, w, atol=2e-4, rtol=2e-5, err_msg=f"after layer {i}")


@pytest.mark.parametrize("name, dtype", [(n, "float32") for n in sorted(lu.CONFIGS)] + [("odd", "bfloat16"), ("even", "bfloat16")])
def test_whole_prompt_and_token_by_token(name, dtype, tmp_path_factory):
    model = _model(name, tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, dtype)
    for n, seed in [(1, 1), (2, 2), (53, 3)]:                      # the first tokens of a sequence; page and window borders and beyond
        toks = _tokens(cfg, n, seed)
        want = _want(model, toks)
        got = zu.run_schedule(eng, {"r": toks}, [[("r", n)]])["r"]
        assert_logits_close(got, want, dtype, f"{name} whole {n}")
        got = zu.run_schedule(eng, {"r": toks}, [[("r", 1)] for _ in range(n)])["r"]
        assert_logits_close(got, want, dtype, f"{name} token by token {n}")


def test_sizes_that_fit_no_vector_width_run_in_bfloat16_too(tmp_path_factory):
    model = _model("ragged", tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, "bfloat16")
    toks = _tokens(cfg, 41, 5)
    want = _want(model, toks)
    whole = zu.run_schedule(eng, {"r": toks}, [[("r", 41)]])["r"]
    cut = zu.run_schedule(eng, {"r": toks}, [[("r", 17)], [("r", 2)], [("r", 21)], [("r", 1)]])["r"]
    assert np.isfinite(whole).all()
    assert np.abs(whole - want).mean() <= 0.05 * want.std()
    assert np.abs(whole - cut).mean() <= 0.03 * want.std()


@pytest.mark.parametrize("name", ["odd", "even", "plain"])
def test_portions_of_every_size(name, tmp_path_factory):
    model = _model(name, tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, "float32")
    toks = _tokens(cfg, 83, 7)
    want = _want(model, toks)
    for sizes in ([2] * 41 + [1], [3, 2, 16, 1, 15, 17, 2, 2, 25], [16, 16, 16, 16, 16, 3], [31, 2, 33, 17], [1, 82]):
        assert sum(sizes) == len(toks)
        got = zu.run_schedule(eng, {"r": toks}, [[("r", k)] for k in sizes])["r"]
        assert_logits_close(got, want, "float32", f"{name} portions {sizes[:4]}...")


@pytest.mark.parametrize("name, dtype", [("odd", "float32"), ("even", "float32"), ("even", "bfloat16"), ("plain", "float32")])
def test_mixed_batches_equal_each_request_alone(name, dtype, tmp_path_factory):
    """Unequal requests side by side, portions beside single tokens, requests that sit out a step, more requests than
    slots over time and a pool that only holds what is live: slots and pages are freed and used again."""
    model = _model(name, tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, dtype, cache_tokens=192, max_requests=3)
    reqs = {"a": _tokens(cfg, 70, 11), "b": _tokens(cfg, 9, 12), "c": _tokens(cfg, 33, 13), "d": _tokens(cfg, 50, 14),
            "e": _tokens(cfg, 1, 15), "f": _tokens(cfg, 18, 16)}
    schedule = [[("a", 30), ("b", 2)], [("b", 1), ("a", 2), ("c", 16)], [("a", 1), ("b", 1), ("c", 1)],
                [("c", 16), ("b", 5)],                              # b and c end: their slots and pages go back
                [("a", 1)], [("d", 20), ("a", 2)], [("e", 1), ("d", 1), ("a", 1)], [("d", 29), ("a", 1)],
                [("f", 2), ("a", 1)], [("f", 16), ("a", 25)]] + [[("a", 1)]] * 6
    got = zu.run_schedule(eng, reqs, schedule)
    if dtype == "float32":
        want = {k: _want(model, v) for k, v in reqs.items()}
    else:
        # in bfloat16 against the same engine running each request alone, whole: where rounding makes the router pick
        # another expert than float64 does, the recurrent state carries the difference on for many tokens, alone as in the
        # batch (the plain implementation judges bfloat16 in the tests above, the batch in the float32 runs of this one)
        alone = _engine(folder, dtype)
        want = {k: zu.run_schedule(alone, {k: v}, [[(k, len(v))]])[k] for k, v in reqs.items()}
    for k in reqs:
        assert_logits_close(got[k], want[k], dtype, f"{name} mixed, request {k}")
    eng.cache.check_invariants()
    assert len(eng.cache.free_slots) == eng.cache.max_requests


def test_long_decoding_through_recorded_steps(tmp_path_factory):
    """150 tokens one by one: the windows (33 and 48) pass over decoded tokens, pages behind them go back to the pool."""
    model = _model("even", tmp_path_factory)
    cfg, _, folder, _ = model
    eng = _engine(folder, "float32", cache_tokens=256)
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
