"""The decode attention entry point that allocates nothing (csrc/attention_decode_static.h).

It serves callers that cannot hand the kernel scratch memory because they cannot allocate
any: the whole GPU already sits in an arena of theirs, or they run where an allocation is
forbidden or would stall the device.  Its scratch is an array inside the library's device
image.  Here it is called through its exported C symbol, twice in a row with different
inputs, and each result is held against the formula in float64 and against the ordinary
entry point's (which gets scratch from the caller) on the same inputs; free device memory
must not move across a call, and a
launch too large for the built-in array must be refused with a clear error.  The file's
name makes pytest collect it last."""

from __future__ import annotations

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def make_case(seed, H, G, D, lengths, n_pages=40):
    """Cached keys and values of several sequences in scattered pages, one query row each."""
    r = np.random.default_rng(seed)
    free = list(r.permutation(n_pages))
    max_pages = max(-(-n // 64) for n in lengths)
    table = np.full((len(lengths), max_pages), -1, dtype=np.int32)
    kp = (r.standard_normal((n_pages, G, 64, D)) * 0.5).astype(np.float32)
    vp = (r.standard_normal((n_pages, G, 64, D)) * 0.5).astype(np.float32)
    for s, n in enumerate(lengths):
        for i in range(-(-n // 64)):
            table[s, i] = int(free.pop())
    rows = len(lengths) + 1
    row_slot = np.array(list(range(len(lengths))) + [-1], dtype=np.int32)     # the last row is padding
    row_pos = np.array([n - 1 for n in lengths] + [0], dtype=np.int32)
    q = (r.standard_normal((rows, H * D)) * 1.5).astype(np.float32)
    cuda = lambda a, dt=None: (torch.from_numpy(a).cuda().to(dt) if dt else torch.from_numpy(a).cuda())
    return dict(q=cuda(q, torch.bfloat16), k=cuda(kp, torch.bfloat16), v=cuda(vp, torch.bfloat16), table=cuda(table),
                pos=cuda(row_pos), slot=cuda(row_slot), rows=rows, H=H, G=G, D=D, max_pages=max_pages, n_pages=n_pages)


def float64_attention(c, window=0):
    """The formula itself (crates/bc-infer/src/model.rs:448-481) in float64 on the values as
    bfloat16 stores them: every row's heads against its sequence's cached positions."""
    q, k, v = (c[n].float().cpu().numpy().astype(np.float64) for n in ("q", "k", "v"))
    table, pos, slot = (c[n].cpu().numpy() for n in ("table", "pos", "slot"))
    H, G, D = c["H"], c["G"], c["D"]
    out = np.zeros((c["rows"], H, D))
    for r in range(c["rows"]):
        if slot[r] < 0:
            continue
        n = int(pos[r]) + 1
        lo = max(0, n - window) if window > 0 else 0
        where = [(int(table[slot[r], t // 64]), t % 64) for t in range(lo, n)]
        for h in range(H):
            g = h // (H // G)
            keys = np.stack([k[p, g, i] for p, i in where])
            vals = np.stack([v[p, g, i] for p, i in where])
            s = keys @ q[r].reshape(H, D)[h] / np.sqrt(D)
            w = np.exp(s - s.max())
            out[r, h] = (w / w.sum()) @ vals
    return out.reshape(c["rows"], H * D)


def call_static(lib, c, out, splits, window=0):
    fn = lib.bc_attention_decode_static_bf16
    fn.restype = ctypes.c_int
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    return fn(p(c["q"]), ctypes.c_int(c["H"] * c["D"]), p(c["k"]), p(c["v"]), p(c["table"]), p(c["pos"]), p(c["slot"]), p(out),
              ctypes.c_int(c["rows"]), ctypes.c_int(c["H"]), ctypes.c_int(c["G"]), ctypes.c_int(c["D"]), ctypes.c_int(c["max_pages"]),
              ctypes.c_int(c["n_pages"]), ctypes.c_int(window), ctypes.c_float(1.0 / c["D"] ** 0.5), ctypes.c_int(splits),
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_entry_point_matches_the_ordinary_one():
    from borrowed_compute_b200 import ops

    lib = ops.lib()
    cases = [(make_case(1, 32, 8, 128, [700, 64, 1, 65, 300]), 5, 0), (make_case(2, 6, 3, 48, [130, 17, 1000]), 3, 70)]
    for c, splits, window in cases:                           # each head size's first call on a device does set-up work: done here,
        warm = torch.empty((c["rows"], c["H"] * c["D"]), dtype=torch.bfloat16, device="cuda")       # so that every call below is an ordinary one
        assert call_static(lib, c, warm, splits, window) == 0, lib.bc_last_error().decode()
    for i, (c, splits, window) in enumerate(cases):           # two calls in a row; the second reuses what the first left
        want = torch.empty((c["rows"], c["H"] * c["D"]), dtype=torch.bfloat16, device="cuda")
        ops.attention_decode(c["q"], c["H"] * c["D"], c["k"], c["v"], c["table"], c["pos"], c["slot"], want, c["H"], c["G"], c["D"],
                             window=window, splits=splits)
        got = torch.full_like(want, 9.0)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        status = call_static(lib, c, got, splits, window)
        torch.cuda.synchronize()
        assert status == 0, lib.bc_last_error().decode()
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the amount of free device memory"
        assert torch.isfinite(got.float()).all()
        # against the formula in float64 (probabilities are rounded to bfloat16 before they weigh the values)
        ref = float64_attention(c, window)
        assert np.abs(got.float().cpu().numpy() - ref).max() <= 2.0 ** -7 * (1 + np.abs(ref).max())
        # Both run the same kernel with the same split of the work: within the decode kernel's tolerance, and in fact equal.
        assert (got.float() - want.float()).abs().max().item() <= 2.0 ** -7 * (1 + want.float().abs().max().item())
        assert torch.equal(got, want)
        assert torch.all(got[-1] == 0), "a padding row must come out as zeros"
        # one split needs no scratch at all and must agree too
        single = torch.empty_like(want)
        assert call_static(lib, c, single, 1, window) == 0
        torch.cuda.synchronize()
        assert (single.float() - want.float()).abs().max().item() <= 2.0 ** -6 * (1 + want.float().abs().max().item())


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from borrowed_compute_b200 import ops

    lib = ops.lib()
    lib.bc_last_error.restype = ctypes.c_char_p
    c = make_case(3, 32, 8, 128, [64] * 40, n_pages=48)
    out = torch.zeros((c["rows"], 32 * 128), dtype=torch.bfloat16, device="cuda")
    status = call_static(lib, c, out, 16)                   # 41 rows * 32 heads * 16 splits * 130 floats > 2^20
    torch.cuda.synchronize()
    assert status != 0 and b"built-in array holds" in lib.bc_last_error()
    assert torch.all(out == 0), "a refused call must not have touched the output"
    assert call_static(lib, c, out, 4) == 0                 # the same rows with fewer splits fit
    torch.cuda.synchronize()
