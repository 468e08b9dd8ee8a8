"""What the parts decide on the host, without a device: which parts a block is made of,
what a mixer may ask of the cache, and the rule that rescales rotary frequencies."""

from __future__ import annotations

import math

import numpy as np
import pytest

import plain_llama
from borrowed_compute_b200.parts import BLOCKS, NORMS, CacheNeed, LayerSpec, PartSpec
from borrowed_compute_b200.parts.rope import inverse_frequencies, llama3_scaled_frequency
from conftest import TINY_B


def test_a_block_names_its_own_parts():
    norm = PartSpec("rmsnorm", {"size": 8, "eps": 1e-5}, "n.")
    att = PartSpec("gqa_attention", {"hidden_size": 8, "heads": 1, "kv_heads": 1, "head_dim": 16, "position": {"kind": "none"}}, "a.")
    ff = PartSpec("swiglu", {"hidden_size": 8, "intermediate_size": 24}, "f.")
    cls = BLOCKS.get("prenorm")
    assert list(cls.ROLES) == ["norm1", "mixer", "norm2", "feed_forward"]
    spec = LayerSpec("prenorm", norm1=norm, mixer=att, norm2=PartSpec("rmsnorm", {"size": 8, "eps": 1e-5}, "m."), feed_forward=ff)
    block = cls.build(spec, 8)
    assert [prefix for prefix, _ in block.named_parts(spec)] == ["n.", "a.", "m.", "f."]
    assert block.memory_part() is block.mixer and isinstance(block.norm1, NORMS.get("rmsnorm"))
    with pytest.raises(ValueError, match="missing \\['norm2'\\].*unexpected \\['norm3'\\]"):
        cls.build(LayerSpec("prenorm", norm1=norm, mixer=att, norm3=norm, feed_forward=ff), 8)
    with pytest.raises(TypeError):
        LayerSpec("prenorm", norm1="rmsnorm")


def test_cache_need_is_planes_of_values_a_position():
    kv = CacheNeed.keys_values(2, 16, window=70)
    assert kv.planes == ((2, 16), (2, 16)) and kv.values_per_token() == 64 and kv.window == 70
    latent = CacheNeed(((1, 24),))
    assert latent.values_per_token() == 24 and latent.key() != kv.key()
    assert CacheNeed(((2, 16), (2, 16)), 70).key() == kv.key()          # equal needs share a storage group
    with pytest.raises(ValueError):
        CacheNeed(())
    with pytest.raises(ValueError):
        CacheNeed(((0, 4),))


def test_the_rotary_part_scales_frequencies_as_the_plain_implementation_does():
    scaling = TINY_B["rope_scaling"]
    got = inverse_frequencies(32, 500000.0, scaling).numpy()
    assert np.array_equal(got, plain_llama.rope_inv_freq(32, 500000.0, scaling))
    assert np.array_equal(inverse_frequencies(32, 500000.0, None).numpy(), plain_llama.rope_inv_freq(32, 500000.0, None))
    # the rule on numbers worked by hand: original 64 positions, factor 4, low 1, high 4
    f_short, f_long, f_mid = 2 * math.pi / 10.0, 2 * math.pi / 100.0, 2 * math.pi / 32.0
    assert llama3_scaled_frequency(f_short, 4.0, 1.0, 4.0, 64) == f_short                 # wavelength 10 < 64 / 4
    assert llama3_scaled_frequency(f_long, 4.0, 1.0, 4.0, 64) == f_long / 4.0             # wavelength 100 > 64 / 1
    t = (64 / 32.0 - 1.0) / (4.0 - 1.0)                                                   # wavelength 32 lies between
    assert abs(llama3_scaled_frequency(f_mid, 4.0, 1.0, 4.0, 64) - ((1 - t) * f_mid / 4.0 + t * f_mid)) < 1e-15
    # continuous at both edges
    for edge in (16.0, 64.0):
        lo, hi = (llama3_scaled_frequency(2 * math.pi / (edge * k), 4.0, 1.0, 4.0, 64) * edge * k for k in (1 - 1e-9, 1 + 1e-9))
        assert abs(lo - hi) < 1e-6
    with pytest.raises(ValueError, match="not known"):
        inverse_frequencies(32, 1e4, {"rope_type": "yarn", "factor": 2.0})
    with pytest.raises(ValueError, match="inconsistent"):
        inverse_frequencies(32, 1e4, {"rope_type": "llama3", "factor": 2.0, "low_freq_factor": 4.0, "high_freq_factor": 1.0,
                                      "original_max_position_embeddings": 64})


def test_how_the_decode_attention_is_cut_into_splits(monkeypatch):
    """The split counts that were measured best on 148 SMs, pinned: few blocks are cut until they
    fill the SMs, by powers of two up to a cluster of eight; one sequence of eight kv heads
    takes a cluster of sixteen from 64 pages on; beyond 192 pages (320 where sixteen serve)
    clusters of eight whose sums go through scratch memory.  (Pages are 64 positions.)"""
    from borrowed_compute_b200 import ops

    monkeypatch.setattr(ops, "sm_count", lambda: 148)
    splits = ops.attention_decode_splits
    assert splits(64, 8, 33) == 1 and splits(16, 8, 33) == 2 and splits(8, 8, 33) == 4     # 512, 128 and 64 blocks before cutting
    assert splits(5, 8, 33) == 4 and splits(7, 8, 33) == 4                                  # 7 and 5 would fill better but place badly
    assert splits(1, 8, 33) == 8 and splits(1, 8, 64) == 8                                  # one sequence of up to 4,096 positions
    assert splits(1, 8, 128) == 16 and splits(1, 8, 320) == 16                              # 8,192 to 20,480: one cluster of sixteen
    assert splits(1, 8, 512) == 32 and splits(1, 8, 2048) == 32                             # beyond: four clusters of eight
    assert splits(2, 8, 128) == 8 and splits(2, 8, 512) == 16                               # two sequences: sixteen blocks before cutting
    assert splits(4, 8, 512) == 8                                                           # 32 blocks: eight fill the SMs
    assert splits(1, 8, 3) == 2 and splits(1, 1, 1) == 1                                    # never more than the pages
    assert splits(16, 40, 18) == 1                                                          # every head its own keys: 640 blocks
