"""Each kernel beside its plain C++ twin (csrc/twin/plain_twin.cpp), at sizes the engine's
configurations do not have: norm, products on the tensor cores and on the CUDA cores with
every epilogue, rotary encoding with the cache append, the three attention kernels, the
activation, argmax and the sampler."""

from __future__ import annotations

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
twin = pytest.importorskip("borrowed_compute_b200.twin")

DTYPES = [torch.float32, torch.bfloat16]


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def stored(a, dtype):
    """What the device holds of `a` in `dtype`, back as float32 on the host."""
    return dev(a, dtype).float().cpu().numpy()


def host(t):
    return t.detach().float().cpu().numpy()


def tol(dtype, ref):
    return (2e-5 if dtype == torch.float32 else 2.0 ** -7) * (1 + np.abs(ref).max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_and_activation(dtype):
    from borrowed_compute_b200 import ops

    r = np.random.default_rng(1)
    x, w = r.standard_normal((7, 200)).astype(np.float32), (1 + 0.3 * r.standard_normal(200)).astype(np.float32)
    out = torch.empty((7, 200), dtype=dtype, device="cuda")
    ops.rmsnorm(dev(x), dev(w), out, 3e-6)
    ref = twin.rmsnorm(x, w, 3e-6)
    assert np.abs(host(out) - ref).max() <= tol(dtype, ref)
    gu = r.standard_normal((5, 2 * 88)).astype(np.float32)
    act = torch.empty((5, 88), dtype=dtype, device="cuda")
    ops.swiglu(dev(gu, dtype), act)
    s = stored(gu, dtype)
    ref = twin.swiglu(s[:, :88], s[:, 88:])
    assert np.abs(host(act) - ref).max() <= tol(dtype, ref)


@pytest.mark.parametrize("product", ["tensor cores", "CUDA cores", "CUDA cores in float32"])
@pytest.mark.parametrize("rows", [1, 37, 200])
def test_products_with_every_epilogue(product, rows):
    from borrowed_compute_b200 import ops

    r = np.random.default_rng(rows)
    dtype = torch.float32 if product.endswith("float32") else torch.bfloat16
    fn = ops.gemm_tc if product == "tensor cores" else ops.gemm_simt
    N, K = 150, 264
    x, w = r.standard_normal((rows, K)).astype(np.float32), (r.standard_normal((2 * N, K)) * 0.2).astype(np.float32)
    xs, ws = stored(x, dtype), stored(w, dtype)
    full = twin.linear(xs, ws)
    xd, wd = dev(x, dtype), dev(w, dtype)
    out = torch.empty((rows, 2 * N), dtype=dtype, device="cuda")
    fn(xd, wd, out, ops.EPI_STORE)
    assert np.abs(host(out) - full).max() <= tol(dtype, full)
    f32 = torch.empty((rows, 2 * N), dtype=torch.float32, device="cuda")
    fn(xd, wd, f32, ops.EPI_STORE_F32)
    assert np.abs(host(f32) - full).max() <= 2e-5 * (1 + np.abs(full).max())
    base = r.standard_normal((rows, 2 * N)).astype(np.float32)
    acc = dev(base)
    fn(xd, wd, acc, ops.EPI_ADD_F32)
    assert np.abs(host(acc) - (base + full)).max() <= 2e-5 * (1 + np.abs(full).max())
    act = torch.empty((rows, N), dtype=dtype, device="cuda")
    fn(xd, wd, act, ops.EPI_SWIGLU)
    ref = twin.swiglu(full[:, :N], full[:, N:])
    assert np.abs(host(act) - ref).max() <= tol(dtype, ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("pairing", ["half", "adjacent"])
def test_rotary_append_and_the_three_attention_kernels(dtype, pairing):
    """One sequence of 150 positions: its prompt through rope_append and the prompt kernels,
    its last row through the decode kernels, all against the twin's rope and attention."""
    from borrowed_compute_b200 import ops
    from borrowed_compute_b200.parts.rope import rotary_table

    r = np.random.default_rng(3)
    H, G, D, n = 6, 2, 64, 150
    freqs = twin.inv_freq(D, 10000.0)
    qkv = (r.standard_normal((n, (H + 2 * G) * D)) * 0.8).astype(np.float32)
    s = stored(qkv, dtype)
    q = twin.rope(s[:, :H * D].reshape(n, H, D), range(n), freqs, pairing)
    k = twin.rope(s[:, H * D:(H + G) * D].reshape(n, G, D), range(n), freqs, pairing)
    v = s[:, (H + G) * D:].reshape(n, G, D)
    ref = twin.attention(stored(q, dtype), stored(k, dtype), v).reshape(n, H * D)
    cos_sin = rotary_table(torch.from_numpy(freqs), 256).cuda()
    pages = torch.zeros((5, G, 64, D), dtype=dtype, device="cuda")
    kc, vc = pages.clone(), pages.clone()
    table = torch.tensor([[3, 0, 4, -1]], dtype=torch.int32, device="cuda")
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
    qd = dev(qkv, dtype)
    pos, slot = i32(list(range(n))), i32([0] * n)
    ops.rope_append(qd, cos_sin, pos, slot, table, kc, vc, H, G, D, 1 if pairing == "adjacent" else 0)
    assert np.abs(host(qd[:, :H * D]) - q.reshape(n, H * D)).max() <= tol(dtype, q)
    assert np.abs(host(kc[3, :, :64]).transpose(1, 0, 2) - k[:64]).max() <= tol(dtype, k)       # the first page of the sequence
    out = torch.empty((n, H * D), dtype=dtype, device="cuda")
    ops.attention_rows(qd, (H + 2 * G) * D, kc, vc, table, pos, slot, out, H, G, D)
    assert np.abs(host(out) - ref).max() <= tol(dtype, ref)
    if dtype == torch.bfloat16:
        for use_tc in (False, True):
            out.fill_(9.0)
            ops.attention_prefill(qd, (H + 2 * G) * D, kc, vc, table, i32([0, n]), i32([0]), i32([0]), out, 1, n, H, G, D, use_tc=use_tc)
            assert np.abs(host(out) - ref).max() <= tol(dtype, ref), f"prompt kernel, tcgen05 {use_tc}"
        last = torch.empty((1, H * D), dtype=dtype, device="cuda")
        for splits in (1, 3):
            ops.attention_decode(qd[n - 1:n].contiguous(), (H + 2 * G) * D, kc, vc, table, i32([n - 1]), i32([0]), last, H, G, D, splits=splits)
            assert np.abs(host(last) - ref[n - 1:]).max() <= tol(dtype, ref), f"decode kernel, {splits} splits"


def test_argmax_and_the_sampler():
    from borrowed_compute_b200 import ops

    r = np.random.default_rng(4)
    V = 3001
    scores = (r.standard_normal((6, V)) * 2.5).astype(np.float32)
    scores[2, 1500] = scores[2, 7] = scores[2].max() + 1      # equal maxima: the first wins
    sd = dev(scores)
    out = torch.empty(6, dtype=torch.int32, device="cuda")
    ops.argmax(sd, out)
    assert out.tolist() == [twin.sample(row, 0.0, 1.0, 0, 0) for row in scores]
    settings = [(0.8, 0.9), (1.0, 1.0), (0.0, 1.0), (1.5, 0.5), (0.3, 0.95), (1.0, 0.99)]
    t = dev(np.array([s[0] for s in settings], dtype=np.float32))
    p = dev(np.array([s[1] for s in settings], dtype=np.float32))
    seed = torch.full((6,), 77, dtype=torch.int64, device="cuda")
    same = 0
    for step in (0, 9, 300):
        ops.sample(sd, t, p, seed, torch.full((6,), step, dtype=torch.int32, device="cuda"), out)
        same += sum(int(a == twin.sample(scores[i], settings[i][0], settings[i][1], 77, step)) for i, a in enumerate(out.tolist()))
    assert same >= 17, "at most one draw of eighteen may land within rounding of a boundary"
