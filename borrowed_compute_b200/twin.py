"""The plain C++ twin of the kernels (csrc/twin/plain_twin.cpp) from Python: every part as a
short host loop, and the whole model as their sequence.  It is no part of the path that
serves; it is what kernels and engine are held against, and the timed CPU baseline of the
tiny workloads.  Built with the host compiler at first use."""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
from typing import Any, Dict, List, Mapping, Optional, Sequence

import numpy as np

from .csrc import build as _build

SOURCE = os.path.join(_build.HERE, "twin", "plain_twin.cpp")
LIB_NAME = "libbc_b200_twin.so"
_lib: Optional[ctypes.CDLL] = None


def _compile() -> str:
    with open(SOURCE, "rb") as f:
        stamp = hashlib.sha256(f.read()).hexdigest()
    for d in _build._candidate_dirs():
        try:
            with open(os.path.join(d, "twin_stamp.txt")) as f:
                if f.read().strip() == stamp and os.path.isfile(os.path.join(d, LIB_NAME)):
                    return os.path.join(d, LIB_NAME)
        except OSError:
            pass
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise _build.KernelBuildError("the plain C++ twin is not built and no C++ compiler (g++) was found")
    out_dir = next((d for d in _build._candidate_dirs() if _build._writable_dir(d)), None)
    if out_dir is None:
        raise _build.KernelBuildError(f"no writable folder for the twin's build among {_build._candidate_dirs()}")
    tmp = os.path.join(out_dir, f".{LIB_NAME}.{os.getpid()}")
    res = subprocess.run([cxx, "-O2", "-std=c++17", "-shared", "-fPIC", SOURCE, "-o", tmp], capture_output=True, text=True)
    if res.returncode != 0:
        raise _build.KernelBuildError(f"compiling the plain C++ twin failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, os.path.join(out_dir, LIB_NAME))
    with open(os.path.join(out_dir, "twin_stamp.txt"), "w") as f:
        f.write(stamp + "\n")
    return os.path.join(out_dir, LIB_NAME)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_compile())
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


# ------------------------------------------------------------------------------- the parts
def rmsnorm(x, w, eps: float) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.empty_like(x)
    lib().twin_rmsnorm(_p(x), _p(w), _p(out), ctypes.c_int(x.shape[0]), ctypes.c_int(x.shape[1]), ctypes.c_float(eps))
    return out


def linear(x, w) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.empty((x.shape[0], w.shape[0]), dtype=np.float32)
    lib().twin_linear(_p(x), _p(w), _p(out), ctypes.c_int(x.shape[0]), ctypes.c_int(w.shape[0]), ctypes.c_int(w.shape[1]))
    return out


def inv_freq(head_dim: int, theta: float, scaling: Optional[Mapping[str, Any]] = None) -> np.ndarray:
    out = np.empty(head_dim // 2, dtype=np.float32)
    s = scaling or {}
    lib().twin_inv_freq(ctypes.c_int(head_dim), ctypes.c_double(theta), ctypes.c_double(float(s.get("factor", 0.0))),
                        ctypes.c_double(float(s.get("low_freq_factor", 1.0))), ctypes.c_double(float(s.get("high_freq_factor", 1.0))),
                        ctypes.c_double(float(s.get("original_max_position_embeddings", 1))), _p(out))
    return out


def rope(x, positions, freqs, pairing: str) -> np.ndarray:
    """x [rows, heads, d] rotated by positions[r] * freqs[i]; pairing "half" or "adjacent"."""
    out, pos, fr = _f32(x).copy(), _i32(positions), _f32(freqs)
    rows, heads, d = out.shape
    lib().twin_rope(_p(out), _p(pos), ctypes.c_int(rows), ctypes.c_int(heads), ctypes.c_int(d), _p(fr), ctypes.c_int(1 if pairing == "adjacent" else 0))
    return out


def attention(q, k, v, window: int = 0) -> np.ndarray:
    q, k, v = _f32(q), _f32(k), _f32(v)
    out = np.empty_like(q)
    lib().twin_attention(_p(q), _p(k), _p(v), _p(out), ctypes.c_int(q.shape[0]), ctypes.c_int(q.shape[1]), ctypes.c_int(k.shape[1]),
                         ctypes.c_int(q.shape[2]), ctypes.c_int(window))
    return out


def swiglu(gate, up) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    lib().twin_swiglu(_p(gate), _p(up), _p(out), ctypes.c_longlong(gate.size))
    return out


def sample(scores, temperature: float, top_p: float, seed: int, step: int) -> int:
    s = _f32(scores)
    fn = lib().twin_sample
    fn.restype = ctypes.c_int
    return int(fn(_p(s), ctypes.c_int(s.size), ctypes.c_float(temperature), ctypes.c_float(top_p), ctypes.c_uint64(seed), ctypes.c_uint64(step)))


# ------------------------------------------------------------------------------- the model
class _TwinModel(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("layers", "hidden", "heads", "kv_heads", "head_dim", "intermediate", "vocab", "pairing")] + \
               [("eps", ctypes.c_float), ("inv_freq", ctypes.c_void_p), ("embed", ctypes.c_void_p)] + \
               [(n, ctypes.POINTER(ctypes.c_void_p)) for n in ("ln1", "wq", "wk", "wv", "wo", "ln2", "gate", "up", "down")] + \
               [("norm", ctypes.c_void_p), ("head", ctypes.c_void_p)]


class TwinLlama:
    """A Llama model held as float32 arrays on the host, from a config.json dict and tensors
    by their names in a model folder."""

    NAMES = {"ln1": "input_layernorm.weight", "wq": "self_attn.q_proj.weight", "wk": "self_attn.k_proj.weight", "wv": "self_attn.v_proj.weight",
             "wo": "self_attn.o_proj.weight", "ln2": "post_attention_layernorm.weight", "gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight",
             "down": "mlp.down_proj.weight"}

    def __init__(self, config: Mapping[str, Any], weights: Mapping[str, Any]):
        heads, hidden = int(config["num_attention_heads"]), int(config["hidden_size"])
        self.vocab = int(config["vocab_size"])
        layers = int(config["num_hidden_layers"])
        head_dim = int(config.get("head_dim") or hidden // heads)
        self._keep: List[np.ndarray] = []      # the arrays the struct points into

        def hold(a) -> int:
            arr = _f32(a)
            self._keep.append(arr)
            return arr.ctypes.data

        m = _TwinModel()
        m.layers, m.hidden, m.heads, m.kv_heads = layers, hidden, heads, int(config.get("num_key_value_heads") or heads)
        m.head_dim, m.intermediate, m.vocab = head_dim, int(config["intermediate_size"]), self.vocab
        m.pairing = 1 if config.get("rope_pairing", "half") == "adjacent" else 0
        m.eps = float(config.get("rms_norm_eps", 1e-5))
        m.inv_freq = hold(inv_freq(head_dim, float(config.get("rope_theta", 10000.0)), config.get("rope_scaling")))
        m.embed = hold(weights["model.embed_tokens.weight"])
        for field, name in self.NAMES.items():
            arr = (ctypes.c_void_p * layers)(*[hold(weights[f"model.layers.{l}.{name}"]) for l in range(layers)])
            self._keep.append(arr)
            setattr(m, field, arr)
        m.norm = hold(weights["model.norm.weight"])
        m.head = m.embed if config.get("tie_word_embeddings", False) else hold(weights["lm_head.weight"])
        self._m = m

    def logits(self, tokens: Sequence[int]) -> np.ndarray:
        t = _i32(tokens)
        out = np.empty((t.size, self.vocab), dtype=np.float32)
        fn = lib().twin_logits
        fn.restype = ctypes.c_int
        if fn(ctypes.byref(self._m), _p(t), ctypes.c_int(t.size), _p(out)) != 0:
            raise ValueError("a token is outside the vocabulary")
        return out

    def generate(self, prompt: Sequence[int], max_tokens: int, temperature: float = 0.0, top_p: float = 1.0, seed: int = 0,
                 stops: Sequence[int] = ()) -> List[int]:
        p, st = _i32(prompt), _i32(list(stops))
        out = np.empty(max(max_tokens, 1), dtype=np.int32)
        fn = lib().twin_generate
        fn.restype = ctypes.c_int
        n = fn(ctypes.byref(self._m), _p(p), ctypes.c_int(p.size), ctypes.c_int(max_tokens), ctypes.c_float(temperature), ctypes.c_float(top_p),
               ctypes.c_uint64(seed), _p(st), ctypes.c_int(st.size), _p(out))
        if n < 0:
            raise ValueError("a token is outside the vocabulary")
        return [int(x) for x in out[:n]]
