"""Whole models at further sizes, against the plain implementation: a head size of 48 (the
mma.sync prompt kernel), 64 with five heads a kv head and a tied head, 128 with eight
heads on one kv head (the tcgen05 prompt kernel), 256 and 34 heads on one kv head (beyond
the tiled kernels: the one-warp-a-row kernel); widths, feed-forward sizes and
vocabularies that are no powers of two; prompts of more than 128 tokens (the product on
pairs of SMs) in a batch of two whose shorter request ends earlier, then single tokens.
The engines are made one after another in one process and dropped without ceremony: a
captured step must not be disturbed by an earlier engine being collected."""

from __future__ import annotations

import numpy as np
import pytest

import plain_llama
from conftest import make_weights, seeded_tokens, tolerance, weights_as_stored, write_folder

pytestmark = pytest.mark.gpu

CONFIGS = {
    "head48": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 264, "num_attention_heads": 6,
               "num_key_value_heads": 2, "head_dim": 48, "intermediate_size": 520, "vocab_size": 1001, "rope_theta": 10000.0,
               "rms_norm_eps": 1e-5, "max_position_embeddings": 1024},
    "head64": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 320, "num_attention_heads": 10,
               "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 1000, "vocab_size": 777, "rope_theta": 10000.0,
               "rms_norm_eps": 1e-6, "max_position_embeddings": 1024, "tie_word_embeddings": True},
    "head128": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 1, "hidden_size": 1024, "num_attention_heads": 8,
                "num_key_value_heads": 1, "head_dim": 128, "intermediate_size": 1536, "vocab_size": 515, "rope_theta": 500000.0,
                "rms_norm_eps": 1e-5, "max_position_embeddings": 2048},
    # a head size beyond the tiled bf16 kernels (the one-warp-a-row kernel serves prompts and single tokens)
    "head256": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 200, "num_attention_heads": 2,
                "num_key_value_heads": 1, "head_dim": 256, "intermediate_size": 328, "vocab_size": 401, "rope_theta": 10000.0,
                "rms_norm_eps": 1e-5, "max_position_embeddings": 1024, "rope_pairing": "adjacent"},
    # a width and a feed-forward size that are no multiples of 8: no TMA box starts on a 16-byte boundary there, the products run on CUDA cores
    "odd_widths": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 90, "num_attention_heads": 2,
                   "num_key_value_heads": 1, "head_dim": 48, "intermediate_size": 77, "vocab_size": 203, "rope_theta": 10000.0,
                   "rms_norm_eps": 1e-5, "max_position_embeddings": 1024},
    # more heads on a kv head (34) than the tiled decode kernel takes
    "group34": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 1, "hidden_size": 272, "num_attention_heads": 34,
                "num_key_value_heads": 1, "head_dim": 16, "intermediate_size": 136, "vocab_size": 333, "rope_theta": 10000.0,
                "rms_norm_eps": 1e-6, "max_position_embeddings": 1024},
}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_further_sizes_in_both_types(name, tmp_path):
    from borrowed_compute_b200.engine import Engine, StepEntry

    cfg = CONFIGS[name]
    w = make_weights(cfg, 3, std=0.05, embed_std=1.0, head_std=0.1)
    a, b = seeded_tokens(1, 300, cfg["vocab_size"]), seeded_tokens(2, 141, cfg["vocab_size"])
    for dtype in ("bfloat16", "float32"):
        folder = write_folder(str(tmp_path / dtype), cfg, w, dtype)
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=2048, max_slots=3)   # the engine before it is dropped here
        stored = weights_as_stored(w, dtype)
        ref_a = plain_llama.logits(cfg, stored, a, dtype=np.float32)
        ref_b = plain_llama.logits(cfg, stored, b, dtype=np.float32)
        sa, sb = eng.acquire(), eng.acquire()
        first = eng.step([StepEntry(sa, a[:260], want=tuple(range(260))), StepEntry(sb, b[:130], want=tuple(range(130)))]).cpu().numpy()
        got_a, got_b = [first[:260]], [first[260:]]
        for i in range(40):
            entries = [StepEntry(sa, [a[260 + i]], want=(0,))] + ([StepEntry(sb, [b[130 + i]], want=(0,))] if 130 + i < len(b) else [])
            out = eng.step(entries).cpu().numpy()
            got_a.append(out[:1])
            if len(entries) == 2:
                got_b.append(out[1:])
            if 130 + i == len(b) - 1:
                eng.release(sb)
        eng.release(sa)
        # The plain run is float32 here; allow for its own rounding too.
        tol = 2 * tolerance(dtype, ref_a)
        assert np.abs(np.concatenate(got_a) - ref_a).max() <= tol, f"{name} {dtype}: the longer request"
        assert np.abs(np.concatenate(got_b) - ref_b).max() <= tol, f"{name} {dtype}: the shorter request"
        eng.cache.slots.check()
