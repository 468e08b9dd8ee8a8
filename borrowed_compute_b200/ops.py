"""Python faces of the CUDA launchers: argument checks, then one call into the kernel library.

Every function launches on torch's current CUDA stream and allocates nothing unless it
says so.  There is no CPU path and no library stand-in: a tensor that is not on a CUDA
device, or a kernel library that cannot be loaded, raises.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .csrc import build as _build

PAGE = 64  # tokens per cache page; checked against the library at load

EPI_STORE, EPI_STORE_F32, EPI_ADD_F32, EPI_SWIGLU = 0, 1, 2, 3

_c_int, _c_float, _c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


_checked_page = False


def lib() -> ctypes.CDLL:
    global _checked_page
    handle = _build.load()
    if not _checked_page:
        handle.bc_page_size.restype = _c_int
        if handle.bc_page_size() != PAGE:
            raise KernelError(f"the kernel library pages {handle.bc_page_size()} tokens, the package {PAGE}")
        _checked_page = True
        if os.environ.get("BC_B200_PDL", "1") == "0":
            handle.bc_set_pdl(_c_int(0))
        if os.environ.get("BC_B200_TC_STAGES"):        # measurement knob: cap the GEMM's TMA ring depth
            handle.bc_gemm_tc_set_stage_cap(_c_int(int(os.environ["BC_B200_TC_STAGES"])))
    return handle


def set_pdl(on: bool) -> None:
    """Whether kernels ask for programmatic dependent launch (overlap of a kernel's set-up
    and weight prefetch with the preceding kernel's tail).  On by default."""
    lib().bc_set_pdl(_c_int(1 if on else 0))


def set_gemm_tc_cluster(on: bool) -> None:
    """Whether two to eight splits of a product with few tokens add up inside a thread-block
    cluster (the default) or through scratch memory like all other splits; both give the same
    bits.  For measurements and tests."""
    lib().bc_gemm_tc_set_cluster(_c_int(1 if on else 0))


def set_gemm_tc_pair(on: bool) -> None:
    """Whether products over more than 128 tokens run on pairs of SMs that share a tile
    (cta_group::2, the default) or every block on its own.  For measurements and tests."""
    lib().bc_gemm_tc_set_pair(_c_int(1 if on else 0))


def set_gemm_tc_pair_tokens(n: int) -> None:
    """Tokens a tile of the paired product takes: 0 lets the launcher choose (256 unless a
    narrower tile saves a whole round of tiles), 64, 128, 192 or 256 force it."""
    lib().bc_gemm_tc_set_pair_tokens(_c_int(int(n)))


def _stream() -> _c_void_p:
    return _c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> _c_void_p:
    return _c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def _suffix(dtype: torch.dtype) -> str:
    if dtype == torch.float32:
        return "f32"
    if dtype == torch.bfloat16:
        return "bf16"
    raise KernelError(f"no kernels for {dtype}: float32 and bfloat16 only")


# ------------------------------------------------------------------ the bounds-checked mode
# With BC_B200_BOUNDS_CHECK=1 (or ``bounds_check = True``) every launcher that takes indices
# (tokens, slots, positions, page tables, gathered rows) first brings them to the host and
# holds each against the extent of what it indexes; a bad one raises KernelError naming the
# tensor, the index and the extent, and nothing is launched.  The kernels themselves guard
# tokens, slots and pages on every build; this mode also catches what they would only skip
# (a position past the table, a gathered row past the rows) and what they trust (a slot past
# the table's rows).  It synchronises on every launch, so it is for finding a fault, not for
# serving; an engine built in this mode steps without captured graphs.  It stands in for a
# memory checker run under the kernels, which cannot be had everywhere.
bounds_check = os.environ.get("BC_B200_BOUNDS_CHECK", "0") == "1"


def _bounds(what: str, values: Optional[torch.Tensor], extent: int, count: Optional[int] = None, lowest: int = 0) -> None:
    """Every one of the first ``count`` values lies in [lowest, extent)."""
    if not bounds_check or values is None or torch.cuda.is_current_stream_capturing():
        return
    v = values.reshape(-1)[: values.numel() if count is None else count]
    if v.numel() == 0:
        return
    bad = ((v < lowest) | (v >= extent)).nonzero()
    if bad.numel():
        i = int(bad[0])
        raise KernelError(f"bounds check: {what}[{i}] = {int(v[i])} is outside [{lowest}, {extent})")


def _bounds_paged(who: str, rows: int, row_pos: torch.Tensor, row_slot: torch.Tensor, page_table: torch.Tensor, n_pages: int) -> None:
    """Slots name rows of the page table (or are -1: padding), positions fit the table's
    width, and every page the table names exists."""
    if not bounds_check or torch.cuda.is_current_stream_capturing():
        return
    _bounds(f"{who}: row_slot", row_slot, page_table.shape[0], rows, lowest=-1)
    live = row_slot.reshape(-1)[:rows] >= 0
    _bounds(f"{who}: row_pos", row_pos.reshape(-1)[:rows][live], page_table.shape[1] * PAGE)
    _bounds(f"{who}: page_table", page_table, n_pages, lowest=-1)


launches = 0   # kernels launched through this module since import (a captured graph replays them uncounted)
_KERNELS_PER_CALL = {"bc_argmax": 2}   # launchers that start more than one kernel


# Timing of single launches, for engine.profile.StepProfile: while `timeline` is a list every
# call records CUDA events around itself and appends (class, launcher, start, end).  The
# class is `label` if a part set one for the product it is about to run, else the launcher's.
timeline: Optional[list] = None
label = ""
_CLASS_OF = {
    "bc_embed": "embedding", "bc_rmsnorm": "norm", "bc_swiglu": "activation", "bc_rope_append": "rotary + append",
    "bc_attention_rows": "attention", "bc_attention_decode": "attention", "bc_attention_prefill": "attention",
    "bc_argmax": "sampling", "bc_sample": "sampling", "bc_gemm": "product", "bc_random": "random weights",
}


def _class_of(name: str) -> str:
    if label:
        return label
    for prefix, cls in _CLASS_OF.items():
        if name.startswith(prefix):
            return cls
    return name


def _call(fn, *args) -> None:
    global launches
    launches += _KERNELS_PER_CALL.get(fn.__name__, 1)
    if timeline is not None:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        status = fn(*args)
        end.record()
        timeline.append((_class_of(fn.__name__), fn.__name__, start, end))
    else:
        status = fn(*args)
    if status != 0:
        msg = lib().bc_last_error()
        raise KernelError(f"{fn.__name__} failed ({status}): {msg.decode() if msg else ''}")


def _fn(name: str):
    f = getattr(lib(), name)
    f.restype = _c_int
    return f


# ---------------------------------------------------------------------------------- row-wise

def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> None:
    """out[r, :] = table[tokens[r], :] widened to float32."""
    _need(table, "table")
    _need(tokens, "tokens", torch.int32)
    _need(out, "out", torch.float32)
    rows, (V, E) = tokens.numel(), table.shape
    if out.shape != (rows, E):
        raise KernelError(f"embed: out is {tuple(out.shape)}, wanted {(rows, E)}")
    _bounds("embed: tokens", tokens, V)
    _call(_fn("bc_embed_" + _suffix(table.dtype)), _ptr(table), _ptr(tokens), _ptr(out), _c_int(rows), _c_int(E), _c_int(V), _stream())


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, gather: Optional[torch.Tensor] = None) -> None:
    """out[i] = x[gather[i] or i] * rsqrt(mean(x^2) + eps) * weight; x and weight float32."""
    _need(x, "x", torch.float32)
    _need(weight, "weight", torch.float32)
    _need(out, "out")
    E = x.shape[-1]
    rows = out.shape[0]
    if weight.numel() != E or out.shape[-1] != E:
        raise KernelError(f"rmsnorm: widths differ: x {E}, weight {weight.numel()}, out {out.shape[-1]}")
    if gather is not None:
        _need(gather, "gather", torch.int32)
        if gather.numel() != rows:
            raise KernelError("rmsnorm: gather and out differ in rows")
        _bounds("rmsnorm: gather", gather, x.shape[0])
    elif x.shape[0] != rows:
        raise KernelError("rmsnorm: x and out differ in rows")
    _call(_fn("bc_rmsnorm_" + _suffix(out.dtype)), _ptr(x), _ptr(weight), _ptr(out), _ptr(gather), _c_int(rows), _c_int(E),
          _c_float(eps), _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[r, j] = silu(gate_up[r, j]) * gate_up[r, F + j]."""
    _need(gate_up, "gate_up")
    _need(out, "out", gate_up.dtype)
    rows, F = out.shape
    if gate_up.shape != (rows, 2 * F):
        raise KernelError(f"swiglu: gate_up is {tuple(gate_up.shape)}, wanted {(rows, 2 * F)}")
    _call(_fn("bc_swiglu_" + _suffix(out.dtype)), _ptr(gate_up), _ptr(out), _c_int(rows), _c_int(F), _stream())


def rope_append(qkv: torch.Tensor, cos_sin: Optional[torch.Tensor], row_pos: torch.Tensor, row_slot: torch.Tensor,
                page_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                pairing: int, write_cache: bool = True) -> None:
    """Rotates q and k of the fused projection in place by each row's position and writes
    rotated k and v into the row's cache page.  k_cache, v_cache: [pages, kv_heads, PAGE, head_dim]."""
    _need(qkv, "qkv")
    _need(row_pos, "row_pos", torch.int32)
    _need(row_slot, "row_slot", torch.int32)
    _need(page_table, "page_table", torch.int32)
    _need(k_cache, "k_cache", qkv.dtype)
    _need(v_cache, "v_cache", qkv.dtype)
    rows = qkv.shape[0]
    if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
        raise KernelError(f"rope_append: qkv width {qkv.shape[1]} is not (heads + 2 kv_heads) * head_dim")
    if row_pos.numel() < rows or row_slot.numel() < rows:
        raise KernelError("rope_append: fewer positions or slots than rows")
    n_pages = k_cache.shape[0]
    if tuple(k_cache.shape[1:]) != (kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"rope_append: cache is {tuple(k_cache.shape)}, wanted [pages, {kv_heads}, {PAGE}, {head_dim}]")
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32)
        if tuple(cos_sin.shape[1:]) != (head_dim // 2, 2):
            raise KernelError(f"rope_append: cos_sin is {tuple(cos_sin.shape)}, wanted [positions, {head_dim // 2}, 2]")
    _bounds_paged("rope_append", rows, row_pos, row_slot, page_table, n_pages)
    if cos_sin is not None and bounds_check and not torch.cuda.is_current_stream_capturing():
        _bounds("rope_append: row_pos (against the rotary table)", row_pos.reshape(-1)[:rows][row_slot.reshape(-1)[:rows] >= 0], cos_sin.shape[0])
    _call(_fn("bc_rope_append_" + _suffix(qkv.dtype)), _ptr(qkv), _ptr(cos_sin), _ptr(row_pos), _ptr(row_slot), _ptr(page_table),
          _ptr(k_cache), _ptr(v_cache), _c_int(rows), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(pairing),
          _c_int(page_table.shape[1]), _c_int(n_pages), _c_int(1 if write_cache else 0), _stream())


def random_normal(out: torch.Tensor, key: int, std: float) -> None:
    """out[i] = std * z(key, i) over out's elements in memory order: z a standard normal
    deviate that depends on the 64-bit key and the index alone (weights/random_init.py has
    the host's mirror, which gives the same bits)."""
    _need(out, "out")
    _call(_fn("bc_random_normal_" + _suffix(out.dtype)), _ptr(out), ctypes.c_longlong(out.numel()), ctypes.c_ulonglong(key & ((1 << 64) - 1)),
          _c_float(std), _stream())


# ---------------------------------------------------------------------------------- products

def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int) -> None:
    """out = x @ w.T on the CUDA cores with float accumulation in ascending k.
    EPI_STORE: out in x's type; EPI_STORE_F32: float32; EPI_ADD_F32: out += (float32);
    EPI_SWIGLU: w stacks gate rows on up rows, out[:, j] = silu(g_j) * u_j in x's type."""
    _need(x, "x")
    _need(w, "w", x.dtype)
    M, K = x.shape
    n_w = w.shape[0]
    N = n_w // 2 if epilogue == EPI_SWIGLU else n_w
    if w.shape[1] != K or (epilogue == EPI_SWIGLU and n_w % 2):
        raise KernelError(f"gemm: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    _need(out, "out", torch.float32 if epilogue in (EPI_STORE_F32, EPI_ADD_F32) else x.dtype)
    if tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: out is {tuple(out.shape)}, wanted {(M, N)}")
    _call(_fn("bc_gemm_simt_" + _suffix(x.dtype)), _ptr(x), _ptr(w), _ptr(out), _c_int(M), _c_int(N), _c_int(K), _c_int(epilogue), _stream())


def sm_count() -> int:
    """Streaming multiprocessors of the current device, as the kernel library sees them."""
    return int(_fn("bc_sm_count")())


_tc_workspace = {}
_TC_FILL = float(os.environ.get("BC_B200_TC_FILL", "2"))      # measurement knobs: blocks an SM a split product aims at,
_SWIGLU_SPLIT = os.environ.get("BC_B200_SWIGLU_SPLIT", "1") == "1"
_TC_MIN_K = int(os.environ.get("BC_B200_TC_MIN_K", "4"))       # and the fewest k-steps of 64 a split keeps
TC_SCRATCH_FLOATS = 148 * 256 * 256   # split-K partial tiles: a capacity of 37 MiB (148 tiles of 256 x 256 floats), whatever the device


def _tc_scratch(device: torch.device):
    """Split-K scratch of the tensor-core product, one a device, allocated at first use:
    float partial tiles (any contents) and int counters (zero between launches)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _tc_workspace:
        _tc_workspace[key] = (torch.empty(TC_SCRATCH_FLOATS, dtype=torch.float32, device=device),
                              torch.zeros(4096, dtype=torch.int32, device=device))
    return _tc_workspace[key]


def gemm_tc_accepts(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core product takes these operands (K a multiple of 8, bf16)."""
    return x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def _tc_tiling(T: int, N: int, epilogue: int):
    """(token tile, output rows a block, blocks) the tensor-core product uses; mirrors the launcher."""
    bn = int(_fn("bc_gemm_tc_token_tile")(_c_int(T), _c_int(epilogue)))
    rows = int(_fn("bc_gemm_tc_rows_per_block")(_c_int(T), _c_int(N), _c_int(epilogue)))
    return bn, rows, -(-N // rows) * -(-T // bn)


def gemm_tc_splits(T: int, N: int, K: int, epilogue: int) -> int:
    """How many ways to split K so that a product with few weight tiles still fills the
    device's SMs: as many as fit, each at least 4 k-steps of 64 (8 measured 3 % slower on the
    3B shape, whose products of K = 3,072 then stopped at 4 splits, and 0.6 % on the 8B shape)."""
    bn, rows, tiles = _tc_tiling(T, N, epilogue)
    if tiles == 0:
        return 1
    sms = sm_count()
    accs = 2 if epilogue == EPI_SWIGLU else 1              # SwiGLU keeps gate and up sums apart until the last split
    fits = TC_SCRATCH_FLOATS // (tiles * accs * rows * bn)   # splits whose partial tiles fit the scratch
    if epilogue == EPI_SWIGLU:
        # The kernel can split SwiGLU (the gate is applied to the full sums), but measured on the
        # 8B shapes two half-depth blocks an SM stream slower than one full-depth block: unsplit,
        # unless the tiles are so few that they leave half of the SMs or more without a block
        # (a feed-forward width of 8,192 is 64 tiles): then one block an SM.
        if bn <= 64 and tiles * 2 <= sms and _SWIGLU_SPLIT:
            s = max(1, min(sms // tiles, -(-K // 64) // _TC_MIN_K, 8, fits))   # two blocks an SM measured slower here too
            return 1 << (s.bit_length() - 1)
        return 1
    if bn <= 64:
        # Few tokens: the product streams weights, two blocks fit an SM, and measured rates keep
        # rising up to about two blocks an SM as long as a split still has a few k-steps of 64.
        s = max(1, min(int(_TC_FILL * sms) // tiles, -(-K // 64) // _TC_MIN_K, 16, fits))
        # Up to eight splits add up inside a thread-block cluster, which saves the trip through
        # scratch memory; clusters of 2, 4 or 8 place well on the SMs, other sizes measured
        # up to 5 us slower.  So a count up to 12 is rounded down to a power of two.
        if s <= 12:
            s = 1 << (min(s, 8).bit_length() - 1)
        return s
    return max(1, min(sms // tiles, -(-K // 64) // 8, 16, fits))


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, splits: Optional[int] = None) -> None:
    """out = x @ w.T for bf16 operands on the tcgen05 tensor cores (float accumulation in
    TMEM), with the epilogues of gemm_simt.  ``splits`` > 1 cuts K across blocks that add
    their partial sums in a fixed order."""
    _need(x, "x", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    M, K = x.shape
    n_w = w.shape[0]
    N = n_w // 2 if epilogue == EPI_SWIGLU else n_w
    if w.shape[1] != K or (epilogue == EPI_SWIGLU and n_w % 2):
        raise KernelError(f"gemm: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    _need(out, "out", torch.float32 if epilogue in (EPI_STORE_F32, EPI_ADD_F32) else torch.bfloat16)
    if tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: out is {tuple(out.shape)}, wanted {(M, N)}")
    if M == 0:
        return
    if splits is None:
        splits = gemm_tc_splits(M, N, K, epilogue)
    partial = counters = None
    if splits > 1:
        partial, counters = _tc_scratch(x.device)
        bn, rows, tiles = _tc_tiling(M, N, epilogue)
        accs = 2 if epilogue == EPI_SWIGLU else 1
        if tiles * splits * accs * rows * bn > partial.numel() or tiles * 4 > counters.numel():
            raise KernelError(f"gemm_tc: {tiles} tiles are too many for the split-K scratch; use splits=1")
    _call(_fn("bc_gemm_tc_bf16"), _ptr(x), _ptr(w), _ptr(out), _c_int(M), _c_int(N), _c_int(K), _c_int(epilogue), _c_int(splits),
          _ptr(partial), _ptr(counters), _stream())


def gemm_tc_status(reset: bool = True) -> int:
    """Waits for the device and returns the tensor-core kernels' status word: 0, or
    (code << 16 | block) of the first bounded wait that gave up."""
    return int(_fn("bc_gemm_tc_status")(_c_int(1 if reset else 0)))


def set_wait_cycles(cycles: int = 0) -> None:
    """The most clocks a bounded wait inside the tensor-core kernels may take before it gives
    up and records its status (0: back to the default, about a second)."""
    for unit in ("gemm_tc", "attention_prefill_tc", "attention_decode"):
        st = _fn(f"bc_{unit}_set_wait_cycles")(ctypes.c_longlong(int(cycles)))
        if st != 0:
            raise KernelError(f"setting the wait limit of {unit} failed ({st})")


def gemm_tc_test_starve_next_launch() -> None:
    """Test hook: the next product of at most 128 tokens waits for bytes that never come, so
    that one of its bounded waits runs out (see csrc/gemm_tc.cu).  Its output stays unwritten."""
    lib().bc_gemm_tc_test_starve_next_launch()


# ------------------------------------------------------------ errors that reach the caller

_STATUS_UNITS = ("the tensor-core product (gemm_tc)", "the tcgen05 prompt attention (attention_prefill_tc)", "the decode attention (attention_decode)")
_WAITS = {
    0: {1: "the loader's wait for a free stage", 2: "the wait for a stage's operands", 3: "the epilogue's wait for the accumulator",
        4: "the wait for the epilogue to hand the accumulator back"},
    1: {1: "the loader's wait for a free stage", 2: "the wait for the queries", 3: "the wait for the first pages", 4: "the wait for P",
        5: "the wait for a page", 6: "the softmax's wait for scores", 7: "the wait for a product that frees P", 8: "the wait for the last product",
        9: "the wait before a rescale"},
    2: {1: "the wait for a page of keys and values"},
}
_bound_devices = set()


def bind_status(device: Optional[torch.device] = None) -> None:
    """Gives the kernels of ``device`` their words of host-visible memory (once a device), so
    that check_status can look without waiting for the device."""
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    if index in _bound_devices:
        return
    with torch.cuda.device(index):
        _call(_fn("bc_status_bind"))
    _bound_devices.add(index)


def check_status(device: Optional[torch.device] = None) -> None:
    """Raises KernelError if a bounded wait of a kernel gave up since the last look.  Costs a
    read of host memory; meaningful after the caller has synchronised with the device (the
    word is written by the kernel that gave up, before it ends).  The word is cleared, so
    the next look reports only what happens after this one."""
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    if index not in _bound_devices:
        return
    peek = _fn("bc_status_peek")
    with torch.cuda.device(index):
        for unit, name in enumerate(_STATUS_UNITS):
            word = int(peek(_c_int(unit), _c_int(1)))
            if word != 0:
                code, block = word >> 16, word & 0xFFFF
                raise KernelError(f"{name}: {_WAITS[unit].get(code, 'a wait')} (code {code}) ran out in block {block}; "
                                  f"what that launch should have written is missing, so this step's results are not valid")


_self_checked = set()


def self_check(device: torch.device) -> None:
    """Once a device and process: every epilogue of the tensor-core product, and the CUDA-core
    product, on a 37 x 512 weight with one row and with three, against float64 sums, as the
    reference checks its products before it trusts a GPU (crates/bc-infer/src/gpu/mod.rs:
    181-206, same sizes, same inputs rule, same 1e-3 (1 + |want|) bound; there a failure means
    the CPU serves, here there is no other path, so it raises)."""
    import numpy as np

    index = device.index if device.index is not None else torch.cuda.current_device()
    if index in _self_checked:
        return
    rows_w, cols = 37, 512
    rng = np.random.default_rng(7)
    w = rng.standard_normal((2 * rows_w, cols)).astype(np.float32) * 0.5
    wb = torch.from_numpy(w).to(device=device, dtype=torch.bfloat16)
    w64 = wb.float().cpu().numpy().astype(np.float64)

    def bad(got: torch.Tensor, want: np.ndarray, rel: float = 1e-3) -> bool:
        g = got.float().cpu().numpy().astype(np.float64)
        return (not np.isfinite(g).all()) or bool((np.abs(g - want) > rel * (1.0 + np.abs(want))).any())

    rounded = 2.0 ** -7    # an output that is itself rounded to bfloat16 carries half an ulp of 2^-8 besides
    for n in (1, 3):       # one row and a batch take different paths
        x = (((np.arange(n * cols) * 31 % 97).astype(np.float32) - 48.0) / 50.0).reshape(n, cols)
        xb = torch.from_numpy(x).to(device=device, dtype=torch.bfloat16)
        x64 = xb.float().cpu().numpy().astype(np.float64)
        full = x64 @ w64.T                                                    # [n, 74]: gate rows, then up rows
        gate, up = full[:, :rows_w], full[:, rows_w:]
        for name, product in (("tensor-core", gemm_tc), ("CUDA-core", gemm_simt)):
            stored = torch.empty((n, 2 * rows_w), dtype=torch.bfloat16, device=device)
            product(xb, wb, stored, EPI_STORE)
            scores = torch.empty((n, 2 * rows_w), dtype=torch.float32, device=device)
            product(xb, wb, scores, EPI_STORE_F32)
            added = torch.full((n, 2 * rows_w), 0.25, dtype=torch.float32, device=device)
            product(xb, wb, added, EPI_ADD_F32)
            gated = torch.empty((n, rows_w), dtype=torch.bfloat16, device=device)
            product(xb, wb, gated, EPI_SWIGLU)
            checks = {"store": bad(stored, full, rounded), "store_f32": bad(scores, full), "add_f32": bad(added, full + 0.25),
                      "swiglu": bad(gated, gate / (1.0 + np.exp(-gate)) * up, rounded)}
            wrong = [k for k, v in checks.items() if v]
            if wrong:
                raise KernelError(f"self-check: the {name} product with {n} row(s) is wrong for the epilogue(s) {wrong} on a "
                                  f"{rows_w} x {cols} weight; this device or this build of the kernels cannot be trusted")
    x = (((np.arange(3 * cols) * 31 % 97).astype(np.float32) - 48.0) / 50.0).reshape(3, cols)
    scores = torch.empty((3, 2 * rows_w), dtype=torch.float32, device=device)
    gemm_simt(torch.from_numpy(x).to(device), torch.from_numpy(w).to(device), scores, EPI_STORE_F32)
    if bad(scores, x.astype(np.float64) @ w.astype(np.float64).T):
        raise KernelError("self-check: the float32 CUDA-core product is wrong; this device or this build of the kernels cannot be trusted")
    torch.cuda.synchronize(device)
    check_status(device)
    _self_checked.add(index)


def set_attention_prefill_tc_tiles(n: int) -> None:
    """Query tiles (of 128 rows) a block of the tcgen05 prompt attention: 0 lets the launcher
    choose (two, unless no sequence brings more rows than one tile holds), 1 or 2 force it.
    For measurements and tests."""
    lib().bc_attention_prefill_tc_set_tiles(_c_int(int(n)))


def attention_prefill_tc_status(reset: bool = True) -> int:
    """The same word of the tcgen05 prompt attention kernel."""
    return int(_fn("bc_attention_prefill_tc_status")(_c_int(1 if reset else 0)))


# --------------------------------------------------------------------------------- attention

def attention_rows(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor,
                   row_pos: torch.Tensor, row_slot: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                   window: int = 0, scale: Optional[float] = None) -> None:
    """Causal attention of every row against its slot's cached positions, one warp a (row, head)."""
    _need(q, "q")
    _need(k_cache, "k_cache", q.dtype)
    _need(v_cache, "v_cache", q.dtype)
    _need(page_table, "page_table", torch.int32)
    _need(row_pos, "row_pos", torch.int32)
    _need(row_slot, "row_slot", torch.int32)
    _need(out, "out", q.dtype)
    rows = out.shape[0]
    if out.shape[1] != heads * head_dim:
        raise KernelError(f"attention: out width {out.shape[1]} is not heads * head_dim")
    if tuple(k_cache.shape[1:]) != (kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention: cache is {tuple(k_cache.shape)}, wanted [pages, {kv_heads}, {PAGE}, {head_dim}]")
    if scale is None:
        scale = 1.0 / float(head_dim) ** 0.5
    _bounds_paged("attention_rows", rows, row_pos, row_slot, page_table, k_cache.shape[0])
    _call(_fn("bc_attention_rows_" + _suffix(q.dtype)), _ptr(q), _c_int(q_stride), _ptr(k_cache), _ptr(v_cache), _ptr(page_table),
          _ptr(row_pos), _ptr(row_slot), _ptr(out), _c_int(rows), _c_int(heads), _c_int(kv_heads), _c_int(head_dim),
          _c_int(page_table.shape[1]), _c_int(k_cache.shape[0]), _c_int(window), _c_float(scale), _stream())


_decode_scratch = {}


def set_attention_decode_tma(on: bool) -> None:
    """Whether the decode attention fetches pages by TMA where the head size (64, 128) allows
    (the default) or by cp.async everywhere; both give the same bits.  For measurements and tests."""
    lib().bc_attention_decode_set_tma(_c_int(1 if on else 0))


def set_attention_decode_cluster16(on: bool) -> None:
    """Whether sixteen splits of the decode attention run as one thread-block cluster of
    sixteen where the device places one (the default) or as two clusters of eight whose sums
    go through scratch memory.  For measurements and tests."""
    lib().bc_attention_decode_set_cluster16(_c_int(1 if on else 0))


def attention_decode_accepts(heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the split decode kernel takes these sizes (bf16; at most 16 heads a kv head;
    head size a multiple of 16 up to 128).  Otherwise attention_rows serves."""
    return dtype == torch.bfloat16 and bool(_fn("bc_attention_decode_accepts")(_c_int(heads), _c_int(kv_heads), _c_int(head_dim)))


def attention_decode_splits(rows: int, kv_heads: int, max_pages: int) -> int:
    """Splits of the cached positions so that rows * kv_heads * splits blocks come close to,
    and stay within, one wave of two blocks on each SM; never more than a sequence
    can have pages.  Up to eight splits merge inside a thread-block cluster, which costs
    about 4 us less than the merge through scratch memory; so eight is the cap unless the
    batch is so small that eight leave most SMs idle and the sequences are long.  Then:
    sixteen as one cluster of sixteen, where all of these find an SM each (one sequence of
    eight kv heads, from 64 pages on: 13 against 18 us a launch at 8,000 positions); and
    beyond 192 pages (320 where sixteen serve) a multiple of eight: clusters of eight merge
    among themselves and only their sums go through scratch memory (32 against 59 us at
    32,000 positions)."""
    blocks = max(1, rows * kv_heads)
    sms = sm_count()
    fill = max(1, min(2 * sms // blocks, max_pages, 64))
    if fill <= 8 or blocks * 8 >= sms:
        # A power of two: clusters of 3, 5, 6 or 7 blocks place badly once the SMs fill up
        # (five sequences of eight kv heads: 20.7 us with 7 splits, 14.7 us with 4).
        return 1 << (min(fill, 8).bit_length() - 1)
    sixteen = blocks * 16 <= sms and fill >= 16
    if sixteen and 64 < max_pages <= 320:
        return 16
    if max_pages <= 192 or (sixteen and max_pages <= 64):
        return 8
    return fill // 8 * 8


def _decode_workspace(device: torch.device, floats: int, ints: int):
    """Scratch of the split decode kernel, one a device, grown outside of any capture and
    never freed (a captured graph keeps pointing at the buffer it saw)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    held = _decode_scratch.setdefault(key, [])
    for f, c in held:
        if f.numel() >= floats and c.numel() >= ints:
            return f, c
    if torch.cuda.is_current_stream_capturing():
        raise KernelError("attention_decode: scratch memory must exist before a graph is captured (run the step once eagerly)")
    f = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device)
    c = torch.zeros(max(ints, 1 << 14), dtype=torch.int32, device=device)
    held.append((f, c))
    return f, c


def attention_decode(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor,
                     row_pos: torch.Tensor, row_slot: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                     window: int = 0, scale: Optional[float] = None, splits: Optional[int] = None, fuse: int = 0,
                     cos_sin: Optional[torch.Tensor] = None, pairing: int = 0, via_scratch: bool = False,
                     reach: Optional[int] = None) -> None:
    """Attention of one new row a sequence (bf16): the cached positions are split across
    blocks and the heads of a kv head share each read; results are merged in a fixed order.
    Two to eight splits form a thread-block cluster and merge through one another's shared
    memory; more (or ``via_scratch``) merge through scratch memory, with the same result.
    ``fuse`` 1 or 2: ``q`` is the fused projection as the product left it; q is rotated on
    the fly by ``cos_sin`` (None: no rotation), and with 2 the row's rotated key and its
    value are appended to the cache first (what rope_append would have done).  ``reach``:
    a bound on the positions any row reaches (else what the page table can hold); the
    number of splits is chosen by it, no result depends on it."""
    _need(q, "q", torch.bfloat16)
    _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16)
    _need(page_table, "page_table", torch.int32)
    _need(row_pos, "row_pos", torch.int32)
    _need(row_slot, "row_slot", torch.int32)
    _need(out, "out", torch.bfloat16)
    rows = out.shape[0]
    if out.shape[1] != heads * head_dim:
        raise KernelError(f"attention: out width {out.shape[1]} is not heads * head_dim")
    if tuple(k_cache.shape[1:]) != (kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention: cache is {tuple(k_cache.shape)}, wanted [pages, {kv_heads}, {PAGE}, {head_dim}]")
    if scale is None:
        scale = 1.0 / float(head_dim) ** 0.5
    if splits is None:
        pages = page_table.shape[1]
        if reach is not None:
            pages = min(pages, -(-max(1, reach) // PAGE))
        if window > 0:
            pages = min(pages, -(-window // PAGE) + 1)
        splits = attention_decode_splits(rows, kv_heads, pages)
    scratch = counters = None
    if splits > 1:
        scratch, counters = _decode_workspace(q.device, rows * heads * splits * (head_dim + 2), rows * kv_heads)
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32)
        if tuple(cos_sin.shape[1:]) != (head_dim // 2, 2):
            raise KernelError(f"attention_decode: cos_sin is {tuple(cos_sin.shape)}, wanted [positions, {head_dim // 2}, 2]")
        if bounds_check and not torch.cuda.is_current_stream_capturing():
            _bounds("attention_decode: row_pos (against the rotary table)", row_pos.reshape(-1)[:rows][row_slot.reshape(-1)[:rows] >= 0], cos_sin.shape[0])
    _bounds_paged("attention_decode", rows, row_pos, row_slot, page_table, k_cache.shape[0])
    _call(_fn("bc_attention_decode_fused_bf16"), _ptr(q), _c_int(q_stride), _ptr(k_cache), _ptr(v_cache), _ptr(page_table), _ptr(row_pos),
          _ptr(row_slot), _ptr(out), _ptr(scratch), _ptr(counters), _c_int(rows), _c_int(heads), _c_int(kv_heads), _c_int(head_dim),
          _c_int(page_table.shape[1]), _c_int(k_cache.shape[0]), _c_int(window), _c_float(scale), _c_int(splits), _ptr(cos_sin),
          _c_int(pairing), _c_int(fuse + (4 if via_scratch else 0)), _stream())


def attention_prefill_accepts(heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tiled prompt kernel takes these sizes (bf16; at most 64 heads a kv head;
    head size a multiple of 16 up to 128).  Otherwise attention_rows serves."""
    return dtype == torch.bfloat16 and bool(_fn("bc_attention_prefill_accepts")(_c_int(heads), _c_int(kv_heads), _c_int(head_dim)))


def attention_prefill_tc_accepts(heads: int, kv_heads: int, head_dim: int, q: Optional[torch.Tensor] = None, q_stride: int = 0) -> bool:
    """Whether the tcgen05 prompt kernel takes these sizes (head size 64 or 128, at most 128
    heads a kv head) and, if given, this q (16-byte aligned, row stride a multiple of 8)."""
    if not _fn("bc_attention_prefill_tc_accepts")(_c_int(heads), _c_int(kv_heads), _c_int(head_dim)):
        return False
    return q is None or (q.data_ptr() % 16 == 0 and q_stride % 8 == 0)


def attention_prefill(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor,
                      seq_rows: torch.Tensor, seq_slot: torch.Tensor, seq_start: torch.Tensor, out: torch.Tensor, seqs: int, max_new: int,
                      heads: int, kv_heads: int, head_dim: int, window: int = 0, scale: Optional[float] = None,
                      use_tc: Optional[bool] = None) -> None:
    """Causal attention of every sequence's new rows against its cached positions (which
    include the new rows' own keys and values), bf16.  Head sizes 64 and 128 run on the
    tcgen05 tensor cores, 128 query rows a block (scores and output accumulate in TMEM);
    other head sizes on mma.sync tiles, 64 rows a block.  ``use_tc`` forces one or the other."""
    _need(q, "q", torch.bfloat16)
    _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16)
    _need(page_table, "page_table", torch.int32)
    _need(seq_rows, "seq_rows", torch.int32)
    _need(seq_slot, "seq_slot", torch.int32)
    _need(seq_start, "seq_start", torch.int32)
    _need(out, "out", torch.bfloat16)
    if out.shape[1] != heads * head_dim:
        raise KernelError(f"attention: out width {out.shape[1]} is not heads * head_dim")
    if tuple(k_cache.shape[1:]) != (kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention: cache is {tuple(k_cache.shape)}, wanted [pages, {kv_heads}, {PAGE}, {head_dim}]")
    if seq_rows.numel() < seqs + 1 or seq_slot.numel() < seqs or seq_start.numel() < seqs:
        raise KernelError("attention_prefill: fewer sequence entries than sequences")
    if scale is None:
        scale = 1.0 / float(head_dim) ** 0.5
    if bounds_check and not torch.cuda.is_current_stream_capturing():
        _bounds("attention_prefill: seq_slot", seq_slot, page_table.shape[0], seqs, lowest=-1)
        _bounds("attention_prefill: seq_rows", seq_rows, out.shape[0] + 1, seqs + 1)
        live = seq_slot.reshape(-1)[:seqs] >= 0
        ends = (seq_start.reshape(-1)[:seqs] + seq_rows.reshape(-1)[1:seqs + 1] - seq_rows.reshape(-1)[:seqs])[live]
        _bounds("attention_prefill: a sequence's last position + 1", ends, page_table.shape[1] * PAGE + 1)
        _bounds("attention_prefill: page_table", page_table, k_cache.shape[0], lowest=-1)
    if use_tc is None:
        use_tc = attention_prefill_tc_accepts(heads, kv_heads, head_dim, q, q_stride)
    if use_tc:
        _call(_fn("bc_attention_prefill_tc_bf16"), _ptr(q), _c_int(q_stride), _c_int(out.shape[0]), _ptr(k_cache), _ptr(v_cache), _ptr(page_table),
              _ptr(seq_rows), _ptr(seq_slot), _ptr(seq_start), _ptr(out), _c_int(seqs), _c_int(max_new), _c_int(heads), _c_int(kv_heads),
              _c_int(head_dim), _c_int(page_table.shape[1]), _c_int(k_cache.shape[0]), _c_int(window), _c_float(scale), _stream())
        return
    _call(_fn("bc_attention_prefill_bf16"), _ptr(q), _c_int(q_stride), _ptr(k_cache), _ptr(v_cache), _ptr(page_table), _ptr(seq_rows),
          _ptr(seq_slot), _ptr(seq_start), _ptr(out), _c_int(seqs), _c_int(max_new), _c_int(heads), _c_int(kv_heads), _c_int(head_dim),
          _c_int(page_table.shape[1]), _c_int(k_cache.shape[0]), _c_int(window), _c_float(scale), _stream())


# ---------------------------------------------------------------------------------- sampling

def argmax(scores: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the first largest score of row r."""
    _need(scores, "scores", torch.float32)
    _need(out, "out", torch.int32)
    rows, V = scores.shape
    _call(_fn("bc_argmax"), _ptr(scores), _c_int(rows), _c_int(V), _ptr(out), _stream())


def set_sample_blocks_per_row(n: int) -> None:
    """Blocks that share a row of the sampler: 0 lets the launcher choose (eight while all
    rows still run at once, fewer for more rows), 1, 2, 4 or 8 force it.  For measurements and tests."""
    lib().bc_sample_set_blocks_per_row(_c_int(int(n)))


def sample(scores: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, seed: torch.Tensor, step: torch.Tensor,
           out: torch.Tensor) -> None:
    """One draw a row: greedy where temperature <= 0, else temperature / nucleus sampling
    with the draw keyed by (seed, step).  seed is int64 (its bits are the 64-bit seed)."""
    _need(scores, "scores", torch.float32)
    _need(temperature, "temperature", torch.float32)
    _need(top_p, "top_p", torch.float32)
    _need(seed, "seed", torch.int64)
    _need(step, "step", torch.int32)
    _need(out, "out", torch.int32)
    rows, V = scores.shape
    for name, t in (("temperature", temperature), ("top_p", top_p), ("seed", seed), ("step", step), ("out", out)):
        if t.numel() < rows:
            raise KernelError(f"sample: {name} has fewer entries than rows")
    _call(_fn("bc_sample"), _ptr(scores), _c_int(rows), _c_int(V), _ptr(temperature), _ptr(top_p), _ptr(seed), _ptr(step), _ptr(out), _stream())
