"""Which kernel a matrix product and a decode attention go to is decided on the host from sizes alone
(``Kernels._route``, ``_use_pair``, ``decode_splits``). These rules were fitted to measurements at the
projection sizes of the 0.5B, 1.5B and 7B models; the test pins them for those sizes so that a change of a
threshold shows up as a decision that moved. No GPU and no library are needed: the rules read nothing but
their arguments, the object's options and its count of SMs."""
import pytest

import dataclasses

from nanoinfer_b200.config import KernelOptions
from nanoinfer_b200.csrc.lib import Kernels, _EPI

SHAPES = {      # hidden, q heads, kv heads, head dim, intermediate
    "0.5b": (896, 14, 2, 64, 4864),
    "1.5b": (1536, 12, 2, 128, 8960),
    "7b": (3584, 28, 4, 128, 18944),
}


@pytest.fixture()
def rules():
    k = Kernels.__new__(Kernels)          # the decision rules only: nothing is loaded
    k.options = KernelOptions()
    k.sm_count = 148
    return k


def projections(shape):
    hidden, heads, kv, hd, inter = SHAPES[shape]
    return {
        "qkv": ((heads + 2 * kv) * hd, hidden, _EPI["store"], True),
        "o": (hidden, heads * hd, _EPI["add"], False),
        "gate_up": (2 * inter, hidden, _EPI["swiglu"], True),
        "down": (hidden, inter, _EPI["add"], False),
    }


def test_decode_products_of_the_small_model_stream_through_the_small_m_kernel(rules):
    p = projections("0.5b")
    for m in (1, 8):
        assert rules._route(m, *p["qkv"]) == ("smallm", True)           # the norm folded in
        assert rules._route(m, *p["o"]) == ("smallm", False)
        assert rules._route(m, *p["gate_up"]) == ("smallm", False)      # wide output: the norm runs alone
        assert rules._route(m, *p["down"]) == ("tc", False)             # long K: split over CTAs on tcgen05
    assert rules._route(64, *p["qkv"]) == ("smallm", False)
    assert rules._route(64, *p["o"])[0] == "tc" and rules._route(64, *p["gate_up"])[0] == "tc"


def test_decode_products_of_the_large_model_go_to_tcgen05_where_the_weights_are_large(rules):
    p = projections("7b")
    assert rules._route(8, *p["qkv"])[0] == "smallm"
    assert rules._route(8, *p["gate_up"])[0] == "tc"
    assert rules._route(8, *p["down"])[0] == "tc"
    lm_head = (152064, 3584, _EPI["f32"], True)
    assert rules._route(1, *lm_head) == ("tc", False)


def test_prefill_products_go_to_pairs_of_sms_when_there_are_tiles_enough(rules):
    for shape in SHAPES:
        p = projections(shape)
        rows, k, epi, _ = p["gate_up"]
        assert rules._use_pair(2048, rows, k, epi)                       # every gate/up product from 256 tokens on
        assert not rules._use_pair(64, rows, k, epi)
    rows, k, epi, _ = projections("0.5b")["o"]
    assert not rules._use_pair(2048, rows, k, epi)                       # 32 tiles of 256 x 256: the one-CTA kernel
    rows, k, epi, _ = projections("0.5b")["down"]
    assert rules._use_pair(2048, rows, k, epi)                           # the same tiles with K split in two
    for name in ("qkv", "o", "down"):
        rows, k, epi, _ = projections("7b")[name]
        assert rules._use_pair(2048, rows, k, epi)
    rules.options = dataclasses.replace(rules.options, gemm_route="tc")
    assert not rules._use_pair(2048, 9728, 896, _EPI["swiglu"])          # a forced route overrides the rule


def test_decode_attention_splits(rules):
    # TMA kernel: about 256 CTAs, at least four tiles (128 keys for heads of 64, else 64) per CTA
    assert rules.decode_splits(8, 2, 4096, 0, True, 64) == 8
    assert rules.decode_splits(1, 2, 4096, 0, True, 64) == 8
    assert rules.decode_splits(64, 2, 4096, 0, True, 64) == 2
    assert rules.decode_splits(8, 4, 4096, 0, True, 128) == 8
    assert rules.decode_splits(64, 4, 4096, 0, True, 128) == 1
    assert rules.decode_splits(8, 2, 100, 0, True, 64) == 1              # a short context is not split
    assert rules.decode_splits(8, 2, 4096, 512, True, 64) == 1           # nor is a window of 512 keys
    rules.options = dataclasses.replace(rules.options, fixed_decode_splits=5)
    assert rules.decode_splits(8, 2, 4096, 0, True, 64) == 4             # the TMA kernel's clusters: 1, 2, 4, 8, 16, 24, ...
    assert rules.decode_splits(8, 2, 4096, 0, False, 64) == 5
    rules.options = dataclasses.replace(rules.options, fixed_decode_splits=21)
    assert rules.decode_splits(8, 2, 4096, 0, True, 64) == 16
