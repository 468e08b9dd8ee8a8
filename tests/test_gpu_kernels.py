"""Each kernel alone against a plain float64 computation of the same operation, at sizes
other than the engine's: widths that are no power of two, head size 48, ragged lengths."""

from __future__ import annotations

import math

import numpy as np
import pytest

import plain_llama

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def f64(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def rng(seed):
    return np.random.default_rng(seed)


DTYPES = [torch.float32, torch.bfloat16]


def stored(a, dtype):
    """Values as the device holds them in ``dtype``, as float64."""
    return f64(dev(a.astype(np.float32), dtype))


def out_tol(dtype, ref):
    return (1e-5 if dtype == torch.float32 else 2.0 ** -8) * (1.0 + np.abs(ref).max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(dtype):
    from borrowed_compute_b200 import ops

    table = rng(0).standard_normal((37, 50)).astype(np.float32)
    tokens = np.array([0, 36, 5, 5, 17, 99, -1], dtype=np.int32)
    out = torch.full((7, 50), 7.0, dtype=torch.float32, device="cuda")
    ops.embed(dev(table, dtype), dev(tokens), out)
    ref = stored(table, dtype)
    got = f64(out)
    assert np.array_equal(got[:5], ref[tokens[:5]])
    assert np.all(got[5:] == 0.0), "a token outside the table must give zeros, never a wild read"


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm(dtype):
    from borrowed_compute_b200 import ops

    x = (rng(1).standard_normal((37, 200)) * 3).astype(np.float32)
    w = (1 + 0.3 * rng(2).standard_normal(200)).astype(np.float32)
    ref = plain_llama.rms_norm(x.astype(np.float64), w.astype(np.float64), 1e-6)
    out = torch.empty((37, 200), dtype=dtype, device="cuda")
    ops.rmsnorm(dev(x), dev(w), out, 1e-6)
    assert np.abs(f64(out) - ref).max() <= out_tol(dtype, ref)
    gather = np.array([36, 0, 5], dtype=np.int32)
    out = torch.empty((3, 200), dtype=dtype, device="cuda")
    ops.rmsnorm(dev(x), dev(w), out, 1e-6, dev(gather))
    assert np.abs(f64(out) - ref[gather]).max() <= out_tol(dtype, ref)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    from borrowed_compute_b200 import ops

    gu = (rng(3).standard_normal((5, 2 * 176)) * 2).astype(np.float32)
    g, u = stored(gu, dtype)[:, :176], stored(gu, dtype)[:, 176:]
    ref = g / (1 + np.exp(-g)) * u
    out = torch.empty((5, 176), dtype=dtype, device="cuda")
    ops.swiglu(dev(gu, dtype), out)
    assert np.abs(f64(out) - ref).max() <= out_tol(dtype, ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(37, 70, 176), (1, 130, 51), (65, 64, 96), (3, 5, 1024)])
def test_gemm_simt(dtype, M, N, K):
    """Odd row counts (the reference self-checks 37 rows, gpu/mod.rs:181-206), K with and
    without the vector path, all four epilogues."""
    from borrowed_compute_b200 import ops

    x = rng(4).standard_normal((M, K)).astype(np.float32)
    w = (rng(5).standard_normal((2 * N, K)) / math.sqrt(K)).astype(np.float32)
    xs, ws = stored(x, dtype), stored(w, dtype)
    full = xs @ ws.T
    xd, wd = dev(x, dtype), dev(w, dtype)
    out = torch.empty((M, N), dtype=dtype, device="cuda")
    ops.gemm_simt(xd, wd[:N].contiguous(), out, ops.EPI_STORE)
    assert np.abs(f64(out) - full[:, :N]).max() <= out_tol(dtype, full)
    out32 = torch.empty((M, N), dtype=torch.float32, device="cuda")
    ops.gemm_simt(xd, wd[:N].contiguous(), out32, ops.EPI_STORE_F32)
    assert np.abs(f64(out32) - full[:, :N]).max() <= 1e-5 * (1 + np.abs(full).max())
    base = rng(6).standard_normal((M, N)).astype(np.float32)
    acc = dev(base)
    ops.gemm_simt(xd, wd[:N].contiguous(), acc, ops.EPI_ADD_F32)
    assert np.abs(f64(acc) - (base + full[:, :N])).max() <= 1e-5 * (1 + np.abs(full).max())
    g, u = full[:, :N], full[:, N:]
    ref = g / (1 + np.exp(-g)) * u
    ops.gemm_simt(xd, wd, out, ops.EPI_SWIGLU)
    assert np.abs(f64(out) - ref).max() <= out_tol(dtype, ref)


def poison(kp, vp, table, lengths, drop_before=None):
    """Everything in the pool that belongs to no position of any sequence becomes
    not-a-number: pages nobody holds, and what lies past a sequence's end in its last page
    (a sequence that held the page before may have left anything there).  ``drop_before[s]``
    also takes the pages wholly before that position away from sequence s (as a windowed
    cache gives them back) and poisons them.  A kernel must not let any of it near a result."""
    owned = np.zeros(kp.shape[:1] + (64,), dtype=bool)
    for s, n in enumerate(lengths):
        first = 0 if drop_before is None else (drop_before[s] // 64)
        for i in range(-(-n // 64)):
            if i < first:
                table[s, i] = -1
                continue
            owned[table[s, i], : min(64, n - 64 * i)] = True
    for a in (kp, vp):
        a[~owned[:, None, :].repeat(a.shape[1], axis=1)] = np.nan
    return kp, vp


def paged(values, page_ids, G, D, n_pages, dtype):
    """Lays values [tokens, G, D] of one sequence out in pages [n_pages, G, 64, D]."""
    pages = np.zeros((n_pages, G, 64, D), dtype=np.float32)
    for t in range(values.shape[0]):
        pages[page_ids[t // 64], :, t % 64, :] = values[t]
    return pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("pairing", ["half", "adjacent"])
def test_rope_append(dtype, pairing):
    from borrowed_compute_b200 import ops
    from borrowed_compute_b200.parts.rope import inverse_frequencies, rotary_table

    H, G, D, n_pages, max_pages = 6, 3, 48, 9, 4
    rows = 7
    pos = np.array([0, 1, 63, 64, 130, 5, 200], dtype=np.int32)
    slot = np.array([0, 1, 0, 1, 2, -1, 2], dtype=np.int32)
    table = np.full((3, max_pages), -1, dtype=np.int32)
    table[0, :1], table[1, :2], table[2, :4] = [4], [7, 2], [1, 8, 3, 0]
    qkv = rng(7).standard_normal((rows, (H + 2 * G) * D)).astype(np.float32)
    inv_freq = inverse_frequencies(D, 10000.0, None)
    assert np.array_equal(inv_freq.numpy(), plain_llama.rope_inv_freq(D, 10000.0, None))
    cos_sin = rotary_table(inv_freq, 256)
    qd = dev(qkv, dtype)
    k_pages = torch.zeros((n_pages, G, 64, D), dtype=dtype, device="cuda")
    v_pages = torch.zeros_like(k_pages)
    ops.rope_append(qd, cos_sin.cuda(), dev(pos), dev(slot), dev(table), k_pages, v_pages, H, G, D, 0 if pairing == "half" else 1)
    src = stored(qkv, dtype).reshape(rows, H + 2 * G, D)
    rot = plain_llama.rope(src[:, :H + G, :], pos, inv_freq.numpy(), pairing)
    got = f64(qd).reshape(rows, H + 2 * G, D)
    tol = out_tol(dtype, src)
    live = slot >= 0
    assert np.abs(got[live, :H] - rot[live, :H]).max() <= tol
    assert np.array_equal(got[~live], src[~live]), "a padding row was touched"
    kp, vp = f64(k_pages), f64(v_pages)
    expect_k, expect_v = np.zeros_like(kp), np.zeros_like(vp)
    for r in range(rows):
        if slot[r] < 0:
            continue
        page = table[slot[r], pos[r] // 64]
        expect_k[page, :, pos[r] % 64, :] = rot[r, H:H + G]
        expect_v[page, :, pos[r] % 64, :] = src[r, H + G:]
    assert np.abs(kp - expect_k).max() <= tol
    assert np.array_equal(vp, expect_v)


@pytest.mark.parametrize("H,G,D", [(6, 3, 48), (4, 4, 16), (32, 8, 128), (5, 1, 64)])
@pytest.mark.parametrize("pairing", [0, 1])
def test_rope_append_of_many_rows_gives_the_bits_of_few_rows(H, G, D, pairing):
    """Prompts of bf16 take a kernel with wider accesses (more than 64 rows a launch): the
    same rows fed 50 at a time go through the narrow kernel and must leave the same bits in
    q and in both caches; padding rows stay untouched."""
    from borrowed_compute_b200 import ops
    from borrowed_compute_b200.parts.rope import inverse_frequencies, rotary_table

    rows, n_pages, max_pages = 150, 12, 4
    r = rng(H + D + pairing)
    slot = r.integers(0, 3, rows).astype(np.int32)
    slot[[3, 77, 149]] = -1
    pos = np.zeros(rows, dtype=np.int32)
    seen = {0: 0, 1: 0, 2: 0}
    for i in range(rows):
        if slot[i] >= 0:
            pos[i] = seen[int(slot[i])]
            seen[int(slot[i])] += 1
    table = np.array([[4, 7, 2, 9], [1, 8, 3, 0], [5, 10, 11, 6]], dtype=np.int32)
    qkv = r.standard_normal((rows, (H + 2 * G) * D)).astype(np.float32)
    cos_sin = rotary_table(inverse_frequencies(D, 10000.0, None), 256).cuda()
    results = []
    for chunk in (rows, 50):
        qd = dev(qkv, torch.bfloat16)
        k_pages = torch.zeros((n_pages, G, 64, D), dtype=torch.bfloat16, device="cuda")
        v_pages = torch.zeros_like(k_pages)
        for a in range(0, rows, chunk):
            ops.rope_append(qd[a:a + chunk], cos_sin, dev(pos[a:a + chunk]), dev(slot[a:a + chunk]), dev(table), k_pages, v_pages, H, G, D, pairing)
        results.append((qd, k_pages, v_pages))
    for wide, narrow, what in zip(results[0], results[1], ("q", "k cache", "v cache")):
        assert torch.equal(wide, narrow), what
    assert torch.equal(results[0][0][[3, 77, 149]], dev(qkv, torch.bfloat16)[[3, 77, 149]]), "a padding row was touched"


def attention_reference(q, k, v, window=0):
    """q [H, D] at the last position of k, v [T, G, D]."""
    H, D = q.shape
    T, G, _ = k.shape
    lo = max(0, T - window) if window > 0 else 0
    out = np.zeros((H, D))
    for h in range(H):
        g = h // (H // G)
        s = k[lo:, g, :] @ q[h] / math.sqrt(D)
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ v[lo:, g, :]
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 20])
@pytest.mark.parametrize("H,G,D", [(6, 3, 48), (2, 1, 256), (4, 2, 160), (34, 1, 16)])
def test_attention_rows(dtype, window, H, G, D):
    """Rows of five sequences of lengths around the page and tile edges, pages scattered; head
    sizes up to the largest the kernel takes (256) and more heads on a kv head than the tiled
    kernels take (34)."""
    from borrowed_compute_b200 import ops

    n_pages = 16
    lengths = [1, 32, 64, 65, 200]
    r = rng(8)
    page_lists = [[5], [9], [2], [11, 0], [7, 3, 14, 1]]
    table = np.full((6, 4), -1, dtype=np.int32)
    kp = np.zeros((n_pages, G, 64, D), dtype=np.float32)
    vp = np.zeros_like(kp)
    ks, vs = [], []
    for s, (n, pages) in enumerate(zip(lengths, page_lists)):
        table[s, :len(pages)] = pages
        k, v = r.standard_normal((n, G, D)).astype(np.float32), r.standard_normal((n, G, D)).astype(np.float32)
        ks.append(k), vs.append(v)
        kp += paged(k, pages, G, D, n_pages, dtype)
        vp += paged(v, pages, G, D, n_pages, dtype)
    # Rows: the last position of every sequence, two earlier positions of the longest, and padding.
    row_slot = np.array([0, 1, 2, 3, 4, 4, -1, 4], dtype=np.int32)
    row_pos = np.array([0, 31, 63, 64, 199, 63, 0, 128], dtype=np.int32)
    poison(kp, vp, table, lengths)
    q = (r.standard_normal((8, H * D)) * 2).astype(np.float32)
    out = torch.full((8, H * D), 9.0, dtype=dtype, device="cuda")
    ops.attention_rows(dev(q, dtype), H * D, dev(kp, dtype), dev(vp, dtype), dev(table), dev(row_pos), dev(row_slot), out,
                       H, G, D, window=window)
    got = f64(out)
    qs = stored(q, dtype)
    for i in range(8):
        if row_slot[i] < 0:
            assert np.all(got[i] == 0.0)
            continue
        s, p = row_slot[i], row_pos[i]
        ref = attention_reference(qs[i].reshape(H, D), stored(ks[s][:p + 1], dtype), stored(vs[s][:p + 1], dtype), window)
        assert np.abs(got[i].reshape(H, D) - ref).max() <= out_tol(dtype, ref), f"row {i}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key(dtype):
    """Random keys hide a lost position: here one key among 300 matches the query, so the
    output must be that position's value, wherever it lies; and just outside a window it
    must vanish."""
    from borrowed_compute_b200 import ops

    H, G, D, n_pages, T = 2, 1, 16, 8, 300
    table = np.array([[6, 1, 4, 2, 7]], dtype=np.int32)
    for far in (0, 31, 32, 63, 64, 127, 128, 255, 256, 299):
        k = np.zeros((T, G, D), dtype=np.float32)
        v = rng(far).standard_normal((T, G, D)).astype(np.float32)
        k[far, 0, 3] = 100.0
        q = np.zeros((1, H * D), dtype=np.float32)
        q[0, 3] = q[0, D + 3] = 4.0
        args = (dev(paged(k, table[0], G, D, n_pages, dtype), dtype), dev(paged(v, table[0], G, D, n_pages, dtype), dtype), dev(table),
                dev(np.array([T - 1], dtype=np.int32)), dev(np.array([0], dtype=np.int32)))
        out = torch.empty((1, H * D), dtype=dtype, device="cuda")
        ops.attention_rows(dev(q, dtype), H * D, *args, out, H, G, D)
        want = stored(v[far, 0], dtype)
        assert np.abs(f64(out).reshape(H, D) - want).max() <= 2.0 ** -7, f"the key at {far} was not found"
        inside, outside = T - far, T - far - 1
        ops.attention_rows(dev(q, dtype), H * D, *args, out, H, G, D, window=inside)
        assert np.abs(f64(out).reshape(H, D) - want).max() <= 2.0 ** -7, f"window {inside} must still see position {far}"
        if outside > 0:
            ops.attention_rows(dev(q, dtype), H * D, *args, out, H, G, D, window=outside)
            assert np.abs(f64(out).reshape(H, D) - want).max() > 0.05, f"window {outside} must not see position {far}"


@pytest.mark.parametrize("kernel", ["decode_cluster", "decode_scratch", "decode_many_splits", "decode_clusters_of_eight", "prefill_mma", "prefill_tcgen05"])
@pytest.mark.parametrize("D", [64, 128])
def test_tensor_core_attention_finds_one_far_key_and_keeps_every_rows_window(kernel, D):
    """The tiled bf16 kernels against planted keys: one key among 700 matches every query, so
    a row's output is that position's value exactly when the row may see it: not before its
    own position reaches it (the causal edge, row by row), and no longer once it has left
    the row's window (the window's edge, row by row).  Wherever the key lies: first and last
    position of a page, of the cached part, of the new rows."""
    from borrowed_compute_b200 import ops

    H, G, n_pages, T, cached, window = 4, 2, 14, 700, 200, 130
    table = np.array([[9, 1, 12, 4, 2, 7, 0, 11, 5, 13, 3]], dtype=np.int32)
    q_row = np.zeros(H * D, dtype=np.float32)
    for h in range(H):
        q_row[h * D + 3] = 4.0
    for far in (0, 63, 64, 199, 200, 201, 447, 448, 640, 698, 699):
        k = np.zeros((T, G, D), dtype=np.float32)
        v = rng(far).standard_normal((T, G, D)).astype(np.float32)
        k[far, :, 3] = 100.0
        kp, vp = dev(paged(k, table[0], G, D, n_pages, torch.bfloat16), torch.bfloat16), dev(paged(v, table[0], G, D, n_pages, torch.bfloat16), torch.bfloat16)
        want = np.repeat(stored(v[far], torch.bfloat16), H // G, axis=0)     # [H, D]: every head of a kv head finds its value
        for w in (0, window):
            if kernel.startswith("decode"):
                rows = [p for p in (far - 1, far, far + 1, far + window - 1, far + window, T - 1) if 0 <= p < T]
                q = dev(np.tile(q_row, (len(rows), 1)), torch.bfloat16)
                out = torch.empty((len(rows), H * D), dtype=torch.bfloat16, device="cuda")
                splits = {"decode_cluster": 4, "decode_scratch": 4, "decode_many_splits": 11, "decode_clusters_of_eight": 16}[kernel]
                ops.attention_decode(q, H * D, kp, vp, dev(table), dev(np.array(rows, dtype=np.int32)), dev(np.zeros(len(rows), dtype=np.int32)),
                                     out, H, G, D, window=w, splits=splits, via_scratch=kernel == "decode_scratch")
                got = {p: f64(out[i]).reshape(H, D) for i, p in enumerate(rows)}
            else:
                new = T - cached
                q = dev(np.tile(q_row, (new, 1)), torch.bfloat16)
                out = torch.empty((new, H * D), dtype=torch.bfloat16, device="cuda")
                ops.attention_prefill(q, H * D, kp, vp, dev(table), dev(np.array([0, new], dtype=np.int32)), dev(np.array([0], dtype=np.int32)),
                                      dev(np.array([cached], dtype=np.int32)), out, 1, new, H, G, D, window=w, use_tc=kernel == "prefill_tcgen05")
                if kernel == "prefill_tcgen05":
                    assert ops.attention_prefill_tc_status() == 0
                got = {p: f64(out[p - cached]).reshape(H, D) for p in range(cached, T)}
            for p, o in got.items():
                sees = far <= p and (w == 0 or far >= p - w + 1)
                err = np.abs(o - want).max()
                if sees:
                    assert err <= 2.0 ** -7, f"{kernel}: the row at {p} (window {w}) did not find the key at {far}"
                elif p > 0:
                    assert err > 0.05, f"{kernel}: the row at {p} (window {w}) must not see the key at {far}"


@pytest.mark.parametrize("H,G,D", [(6, 3, 48), (4, 4, 16), (16, 1, 32), (32, 8, 128), (8, 2, 64)])
@pytest.mark.parametrize("splits", [1, 3, 8, 10, 11, 12, 16, 24])
@pytest.mark.parametrize("window", [0, 70])
def test_attention_decode(H, G, D, splits, window):
    """The split bf16 decode kernel against the float64 formula and its one-warp twin, for
    lengths around page and tile edges, scattered pages, padding rows."""
    from borrowed_compute_b200 import ops

    n_pages = 24
    lengths = [1, 17, 64, 65, 200, 700]
    r = rng(H * 100 + D)
    free = list(r.permutation(n_pages))
    table = np.full((len(lengths), 12), -1, dtype=np.int32)
    kp = np.zeros((n_pages, G, 64, D), dtype=np.float32)
    vp = np.zeros_like(kp)
    ks, vs = [], []
    for s, n in enumerate(lengths):
        pages = [int(free.pop()) for _ in range((n + 63) // 64)]
        table[s, :len(pages)] = pages
        k, v = r.standard_normal((n, G, D)).astype(np.float32), r.standard_normal((n, G, D)).astype(np.float32)
        ks.append(k), vs.append(v)
        kp += paged(k, pages, G, D, n_pages, torch.bfloat16)
        vp += paged(v, pages, G, D, n_pages, torch.bfloat16)
    row_slot = np.array([0, 1, -1, 2, 3, 4, 5], dtype=np.int32)
    row_pos = np.array([n - 1 for n in lengths[:2]] + [0] + [n - 1 for n in lengths[2:]], dtype=np.int32)
    q = (r.standard_normal((7, H * D)) * 1.5).astype(np.float32)
    # what no position owns is not-a-number; under a window the pages behind it are gone, as in a windowed cache
    poison(kp, vp, table, lengths, drop_before=[max(0, n - window) for n in lengths] if window else None)
    args = (dev(q, torch.bfloat16), H * D, dev(kp, torch.bfloat16), dev(vp, torch.bfloat16), dev(table), dev(row_pos), dev(row_slot))
    out = torch.full((7, H * D), 9.0, dtype=torch.bfloat16, device="cuda")
    twin = torch.empty_like(out)
    ops.attention_decode(*args, out, H, G, D, window=window, splits=splits)
    ops.attention_rows(*args, twin, H, G, D, window=window)
    assert bool(torch.isfinite(out.float()).all()) and bool(torch.isfinite(twin.float()).all())
    if D in (64, 128):     # pages by TMA or by cp.async: the same bits
        ops.set_attention_decode_tma(False)
        try:
            other = torch.empty_like(out)
            ops.attention_decode(*args, other, H, G, D, window=window, splits=splits)
        finally:
            ops.set_attention_decode_tma(True)
        assert torch.equal(out, other), "pages fetched by TMA and by cp.async must give the same bits"
        torch.cuda.synchronize()
        ops.check_status()
    again = torch.empty_like(out)
    ops.attention_decode(*args, again, H, G, D, window=window, splits=splits)
    assert torch.equal(out, again), "the same launch twice must give the same bits"
    again.fill_(5.0)
    ops.attention_decode(*args, again, H, G, D, window=window, splits=splits, via_scratch=True)
    near = lambda a, b: (a.float() - b.float()).abs().max().item() <= 2.0 ** -7 * (1 + b.float().abs().max().item())
    if splits <= 8 or splits % 2 or splits == 16:   # sixteen are one cluster where the device places one
        assert torch.equal(out, again), "splits merged through a cluster's shared memory and through scratch memory must agree"
    else:   # clusters of eight, four or two add their own splits first, then the clusters' sums are added: another order of the same sum
        assert near(out, again)
    if splits == 16:
        ops.set_attention_decode_cluster16(False)
        try:
            ops.attention_decode(*args, again, H, G, D, window=window, splits=splits)
        finally:
            ops.set_attention_decode_cluster16(True)
        assert near(again, out), "two clusters of eight against one of sixteen"
    got, qs = f64(out), stored(q, torch.bfloat16)
    for i in range(7):
        if row_slot[i] < 0:
            assert np.all(got[i] == 0.0)
            continue
        s, p = row_slot[i], row_pos[i]
        ref = attention_reference(qs[i].reshape(H, D), stored(ks[s][:p + 1], torch.bfloat16), stored(vs[s][:p + 1], torch.bfloat16), window)
        # Probabilities are rounded to bf16 before they weigh the values: 2^-8 of the largest value.
        assert np.abs(got[i].reshape(H, D) - ref).max() <= 2.0 ** -7 * (1 + np.abs(ref).max()), f"row {i}"
    assert (out.float() - twin.float()).abs().max().item() <= 2.0 ** -6


def test_tcgen05_prompt_attention_refuses_what_it_cannot_do():
    """Head sizes other than 64 and 128, and a q that is not 16-byte aligned, are for the
    mma.sync kernel: the chooser says so, and forcing the tcgen05 kernel is a clear error."""
    from borrowed_compute_b200 import ops

    assert ops.attention_prefill_tc_accepts(32, 8, 128) and ops.attention_prefill_tc_accepts(10, 2, 64)
    assert not ops.attention_prefill_tc_accepts(6, 2, 48) and not ops.attention_prefill_tc_accepts(8, 3, 64)
    H, G, D = 6, 2, 48
    q = torch.zeros((4, H * D), dtype=torch.bfloat16, device="cuda")
    k = torch.zeros((2, G, 64, D), dtype=torch.bfloat16, device="cuda")
    ints = lambda *v: torch.tensor(v, dtype=torch.int32, device="cuda")
    with pytest.raises(ops.KernelError, match="head size 64 or 128"):
        ops.attention_prefill(q, H * D, k, k.clone(), ints(0, 1).reshape(1, 2), ints(0, 4), ints(0), ints(0), torch.empty_like(q), 1, 4,
                              H, G, D, use_tc=True)
    H, G, D = 4, 2, 64
    buf = torch.zeros((4 * H * D + 8,), dtype=torch.bfloat16, device="cuda")
    shifted = buf[4:4 + 4 * H * D].reshape(4, H * D)                      # 8 bytes off a 16-byte boundary
    assert not ops.attention_prefill_tc_accepts(H, G, D, shifted, H * D)


def run_attention_prefill(H, G, D, window, use_tc, cached, new, q_scale=1.5):
    """One launch of a prompt kernel over sequences that bring new[s] rows after cached[s]
    positions (with a padding sequence among them), against the float64 formula at chosen
    rows and against the one-warp-a-row twin at all rows."""
    from borrowed_compute_b200 import ops

    width = max((c + n + 63) // 64 for c, n in zip(cached, new)) + 1
    n_pages = sum((c + n + 63) // 64 for c, n in zip(cached, new)) + 3
    r = rng(H * 100 + D + 1)
    free = list(r.permutation(n_pages))
    table = np.full((len(new), width), -1, dtype=np.int32)
    kp = np.zeros((n_pages, G, 64, D), dtype=np.float32)
    vp = np.zeros_like(kp)
    ks, vs, qs_ = [], [], []
    for s, (c, n) in enumerate(zip(cached, new)):
        pages = [int(free.pop()) for _ in range((c + n + 63) // 64)]
        table[s, :len(pages)] = pages
        k, v = r.standard_normal((c + n, G, D)).astype(np.float32), r.standard_normal((c + n, G, D)).astype(np.float32)
        ks.append(k), vs.append(v)
        kp += paged(k, pages, G, D, n_pages, torch.bfloat16)
        vp += paged(v, pages, G, D, n_pages, torch.bfloat16)
        qs_.append((r.standard_normal((n, H * D)) * q_scale).astype(np.float32))
    # what no position owns is not-a-number; under a window the pages behind the first new row's window are gone
    poison(kp, vp, table, [c + n for c, n in zip(cached, new)],
           drop_before=[max(0, c + 1 - window) for c in cached] if window else None)
    # sequence order in the step: 0, 1, a padding sequence, then the rest
    order = [0, 1, -1] + list(range(2, len(new)))
    seq_rows, seq_slot, seq_start, rows = [0], [], [], []
    for s in order:
        n = 0 if s < 0 else new[s]
        seq_rows.append(seq_rows[-1] + n)
        seq_slot.append(s)
        seq_start.append(0 if s < 0 else cached[s])
        if s >= 0:
            rows.append(qs_[s])
    q = np.concatenate(rows)
    total = q.shape[0]
    out = torch.full((total, H * D), 9.0, dtype=torch.bfloat16, device="cuda")
    ops.attention_prefill(dev(q, torch.bfloat16), H * D, dev(kp, torch.bfloat16), dev(vp, torch.bfloat16), dev(table),
                          dev(np.array(seq_rows, dtype=np.int32)), dev(np.array(seq_slot, dtype=np.int32)),
                          dev(np.array(seq_start, dtype=np.int32)), out, len(order), max(new), H, G, D, window=window, use_tc=use_tc)
    if use_tc:
        assert ops.attention_prefill_tc_status() == 0
    assert bool(torch.isfinite(out.float()).all()), "something nobody owns reached a result"
    got, qst = f64(out), stored(q, torch.bfloat16)
    at = 0
    for s in order:
        if s < 0:
            continue
        for i in range(new[s]):
            p = cached[s] + i
            if i in (0, 1, new[s] // 2, new[s] - 2, new[s] - 1) or (p % 64) in (0, 63):
                ref = attention_reference(qst[at + i].reshape(H, D), stored(ks[s][:p + 1], torch.bfloat16),
                                          stored(vs[s][:p + 1], torch.bfloat16), window)
                assert np.abs(got[at + i].reshape(H, D) - ref).max() <= 2.0 ** -7 * (1 + np.abs(ref).max()), f"sequence {s} row {i}"
        at += new[s]
    row_slot = np.concatenate([np.full(new[s], s, dtype=np.int32) for s in order if s >= 0])
    row_pos = np.concatenate([np.arange(cached[s], cached[s] + new[s], dtype=np.int32) for s in order if s >= 0])
    twin = torch.empty_like(out)
    ops.attention_rows(dev(q, torch.bfloat16), H * D, dev(kp, torch.bfloat16), dev(vp, torch.bfloat16), dev(table), dev(row_pos),
                       dev(row_slot), twin, H, G, D, window=window)
    assert (out.float() - twin.float()).abs().max().item() <= 2.0 ** -5


@pytest.mark.parametrize("H,G,D", [(6, 2, 48), (4, 4, 16), (8, 1, 32), (32, 8, 128), (8, 2, 64)])
@pytest.mark.parametrize("window", [0, 70])
def test_attention_prefill(H, G, D, window):
    """The mma.sync prompt kernel: sequences of ragged lengths in one launch, some
    continuing from cached positions, a padding sequence, head groups that do and do not
    divide the 64-row tile."""
    run_attention_prefill(H, G, D, window, False, cached=[0, 0, 100, 64, 0], new=[1, 130, 30, 65, 300])


@pytest.mark.parametrize("H,G,D", [(32, 8, 128), (8, 2, 64), (12, 4, 64), (4, 4, 128), (16, 1, 64), (10, 2, 128)])
@pytest.mark.parametrize("window", [0, 70, 200])
@pytest.mark.parametrize("q_scale", [1.5, 8.0])
@pytest.mark.parametrize("tiles", [1, 2])
def test_attention_prefill_on_tcgen05(H, G, D, window, q_scale, tiles):
    """The tcgen05 prompt kernel, one and two query tiles a block, at the same workload and a
    longer one (the ring of pages wraps, both score buffers are reused); head groups of 1, 3,
    4, 5 and 16; large scores, so that the running maximum is raised and the accumulator in
    TMEM rescaled many times."""
    from borrowed_compute_b200 import ops

    try:
        ops.set_attention_prefill_tc_tiles(tiles)
        run_attention_prefill(H, G, D, window, True, cached=[0, 0, 100, 64, 0], new=[1, 130, 30, 65, 300], q_scale=q_scale)
        run_attention_prefill(H, G, D, window, True, cached=[0, 70, 0, 1000, 63], new=[2, 900, 129, 17, 64], q_scale=q_scale)
    finally:
        ops.set_attention_prefill_tc_tiles(0)


@pytest.mark.parametrize("H,G,D", [(6, 3, 48), (4, 4, 16), (16, 1, 32), (32, 8, 128), (8, 2, 64), (40, 40, 128)])
@pytest.mark.parametrize("pairing", [0, 1])
def test_attention_decode_with_rotation_and_append_fused(H, G, D, pairing):
    """fuse=2 on the raw projection must leave the same cache and give the same output,
    to the bit, as rope_append followed by the plain decode kernel."""
    from borrowed_compute_b200 import ops
    from borrowed_compute_b200.parts.rope import inverse_frequencies, rotary_table

    r = rng(H + D + pairing)
    n_pages, lengths = 20, [1, 64, 65, 130, 400]
    free = list(r.permutation(n_pages))
    table = np.full((len(lengths), 8), -1, dtype=np.int32)
    for s, n in enumerate(lengths):
        for i in range(-(-n // 64)):
            table[s, i] = int(free.pop())
    kp_host = (r.standard_normal((n_pages, G, 64, D)) * 0.7).astype(np.float32)
    vp_host = (r.standard_normal((n_pages, G, 64, D)) * 0.7).astype(np.float32)
    # The rows about to be appended (position n - 1 of every sequence) and all that no position
    # owns hold not-a-numbers: the appended row must replace them, the rest must stay away.
    poison(kp_host, vp_host, table, [n - 1 for n in lengths])
    kp, vp = dev(kp_host, torch.bfloat16), dev(vp_host, torch.bfloat16)
    rows = len(lengths) + 1
    row_slot = dev(np.array(list(range(len(lengths))) + [-1], dtype=np.int32))
    row_pos = dev(np.array([n - 1 for n in lengths] + [3], dtype=np.int32))
    qkv = dev((r.standard_normal((rows, (H + 2 * G) * D)) * 1.2).astype(np.float32), torch.bfloat16)
    cos_sin = rotary_table(inverse_frequencies(D, 10000.0, None), 512).cuda()
    tab = dev(table)
    # the two-kernel way
    q1, k1, v1 = qkv.clone(), kp.clone(), vp.clone()
    ops.rope_append(q1, cos_sin, row_pos, row_slot, tab, k1, v1, H, G, D, pairing)
    want = torch.empty((rows, H * D), dtype=torch.bfloat16, device="cuda")
    ops.attention_decode(q1, (H + 2 * G) * D, k1, v1, tab, row_pos, row_slot, want, H, G, D, splits=3)
    # fused
    q2, k2, v2 = qkv.clone(), kp.clone(), vp.clone()
    got = torch.empty_like(want)
    ops.attention_decode(q2, (H + 2 * G) * D, k2, v2, tab, row_pos, row_slot, got, H, G, D, splits=3, fuse=2, cos_sin=cos_sin, pairing=pairing)
    same = lambda a, b: torch.equal(torch.nan_to_num(a.float(), nan=123.0), torch.nan_to_num(b.float(), nan=123.0))
    assert same(k1, k2) and same(v1, v2), "the fused append left another cache"
    assert torch.equal(q2, qkv), "the fused kernel must not write the projection"
    assert bool(torch.isfinite(want[:-1].float()).all()) and torch.equal(got, want)
    if D in (64, 128):
        ops.set_attention_decode_tma(False)
        try:
            q4, k4, v4, other = qkv.clone(), kp.clone(), vp.clone(), torch.empty_like(want)
            ops.attention_decode(q4, (H + 2 * G) * D, k4, v4, tab, row_pos, row_slot, other, H, G, D, splits=3, fuse=2, cos_sin=cos_sin, pairing=pairing)
        finally:
            ops.set_attention_decode_tma(True)
        assert torch.equal(other, got) and same(k4, k2) and same(v4, v2), "pages by TMA and by cp.async"
    # fuse=1 rotates but leaves the cache alone (a run that reads another run's cache)
    k3, v3 = k1.clone(), v1.clone()
    ops.attention_decode(qkv.clone(), (H + 2 * G) * D, k3, v3, tab, row_pos, row_slot, got, H, G, D, splits=2, fuse=1, cos_sin=cos_sin, pairing=pairing)
    assert same(k3, k1) and same(v3, v1)
    ops.attention_decode(q1, (H + 2 * G) * D, k1, v1, tab, row_pos, row_slot, want, H, G, D, splits=2)
    assert torch.equal(got, want)


def test_argmax_first_largest_wins():
    from borrowed_compute_b200 import ops

    scores = rng(9).standard_normal((5, 1001)).astype(np.float32)
    scores[1, [7, 500, 900]] = 50.0
    scores[2, 1000] = 60.0
    scores[3, 0] = 60.0
    scores[4, :] = -3.0
    out = torch.empty(5, dtype=torch.int32, device="cuda")
    ops.argmax(dev(scores), out)
    assert out.cpu().tolist() == [plain_llama.argmax(row) for row in scores] == [int(scores[0].argmax()), 7, 1000, 0, 0]


def run_sampler(scores, temperature, top_p, seed, steps):
    from borrowed_compute_b200 import ops

    n = scores.shape[0]
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    seeds = np.array([seed - (1 << 64) if seed >= (1 << 63) else seed] * n, dtype=np.int64)
    ops.sample(dev(scores), dev(np.full(n, temperature, dtype=np.float32)), dev(np.full(n, top_p, dtype=np.float32)),
               dev(seeds), dev(np.asarray(steps, dtype=np.int32)), out)
    return out.cpu().tolist()


def test_sampler_on_the_reference_case():
    """crates/bc-infer/src/sample.rs:77-89."""
    scores = np.array([[0.1, 3.0, 2.9, -5.0]], dtype=np.float32)
    assert run_sampler(scores, 0.0, 1.0, 0, [0]) == [1]
    rows = np.repeat(scores, 200, axis=0)
    assert set(run_sampler(rows[:20], 1.0, 0.01, 7, range(20))) == {1}
    picks = run_sampler(rows, 1.0, 0.95, 7, range(200))
    assert 1 in picks and 2 in picks and 3 not in picks
    assert picks == run_sampler(rows, 1.0, 0.95, 7, range(200)), "seeded"
    assert picks == [plain_llama.sample(scores[0], 1.0, 0.95, 7, i) for i in range(200)]


@pytest.mark.parametrize("V", [1000, 5003])
@pytest.mark.parametrize("temperature,top_p", [(0.8, 0.9), (1.0, 1.0), (1.5, 0.5), (0.3, 0.95)])
def test_sampler_matches_the_plain_one(V, temperature, top_p):
    """The device picks the token the sorted walk picks.  Where the uniform draw lands
    within rounding of a boundary between two tokens either may be picked; such rows are
    told apart by the margin and must be rare."""
    scale = 3.0 if V == 1000 else 0.5
    scores = (rng(V).standard_normal((64, V)) * scale).astype(np.float32)
    scores[5, 10:20] = scores[5, 3]          # ties: equal weights keep ascending ids
    seed = 0x9E3779B97F4A7C15
    got = run_sampler(scores, temperature, top_p, seed, range(100, 164))
    same = 0
    for r in range(64):
        want = plain_llama.sample(scores[r], temperature, top_p, seed, 100 + r)
        if got[r] == want:
            same += 1
            continue
        order, w = plain_llama.nucleus(scores[r], temperature, top_p)
        assert got[r] in order, f"row {r}: token {got[r]} is outside the nucleus"
        u = plain_llama.uniform((seed ^ (((100 + r) * 0x9E3779B97F4A7C15) & plain_llama.MASK64)) & plain_llama.MASK64) * w.sum()
        cum = np.cumsum(w)
        i = order.index(got[r])
        lo, hi = (cum[i - 1] if i else 0.0), cum[i]
        assert lo - 1e-4 * w.sum() <= u <= hi + 1e-4 * w.sum(), f"row {r}: token {got[r]} does not hold the draw"
    assert same >= 60


def test_sampler_rows_are_independent():
    scores = (rng(11).standard_normal((8, 777)) * 2).astype(np.float32)
    alone = [run_sampler(scores[i:i + 1], 0.9, 0.9, 42, [50 + i])[0] for i in range(8)]
    assert run_sampler(scores, 0.9, 0.9, 42, range(50, 58)) == alone


def test_sampler_on_a_row_too_long_to_keep_in_registers():
    """Past 147,456 scores a thread no longer keeps its weights between the passes and takes
    them from the scores again: the same picks as the plain sampler."""
    V = 150_001
    scores = (rng(V).standard_normal((6, V)) * 3.0).astype(np.float32)
    seed = 12345
    got = run_sampler(scores, 0.9, 0.8, seed, range(40, 46))
    same = sum(got[r] == plain_llama.sample(scores[r], 0.9, 0.8, seed, 40 + r) for r in range(6))
    for r in range(6):
        order, w = plain_llama.nucleus(scores[r], 0.9, 0.8)
        assert got[r] in order
    assert same >= 5


def test_sampler_picks_do_not_depend_on_how_many_blocks_share_a_row():
    from borrowed_compute_b200 import ops

    scores = (rng(21).standard_normal((5, 9001)) * 2.5).astype(np.float32)
    picks = []
    try:
        for share in (8, 4, 2, 1, 0):
            ops.set_sample_blocks_per_row(share)
            picks.append(run_sampler(scores, 0.7, 0.9, 99, range(5)))
    finally:
        ops.set_sample_blocks_per_row(0)
    assert all(p == picks[0] for p in picks)
