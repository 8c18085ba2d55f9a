"""The Python entry point's edges on the host backend: the context limit with and without the cache,
what an error in a step leaves behind, and that a kernel which gave up waiting is reported."""
import dataclasses

import pytest

from tiny_configs import TINY_A
from torch_ops import TorchOps

from nanoinfer_b200.api import Model
from nanoinfer_b200.config import EngineConfig
from nanoinfer_b200.csrc.lib import KernelError, raise_device_errors
from nanoinfer_b200.registry import config_from_json_dict
from nanoinfer_b200.weights import write_random_model


def host_model(model_dir, **kw):
    cfg = EngineConfig(dtype="float32", page_size=4, num_pages=64, max_batch=2, device="cpu", cuda_graphs=False, **kw)
    return Model(model_dir, cfg, ops=TorchOps())


@pytest.fixture(scope="module")
def short_context_dir(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("short_ctx"))
    write_random_model(config_from_json_dict(dict(TINY_A, max_position_embeddings=12)), d, seed=7)
    return d


@pytest.mark.parametrize("prompt_len", [3, 9, 11, 12])
def test_cached_and_recomputed_generation_stop_alike_at_the_context_limit(short_context_dir, prompt_len):
    """max_position_embeddings = 12: both ways emit tokens until the sequence holds 12 ids (one token for a
    prompt that fills the context already), and both give the same tokens."""
    m = host_model(short_context_dir)
    prompt = [(7 * i + 3) % 256 for i in range(prompt_len)]
    cached = m.generate(prompt, max_tokens=40, eos_id=-1)
    recomputed = m.generate(prompt, max_tokens=40, eos_id=-1, use_cache=False)
    assert cached == recomputed
    assert len(cached) == max(1, 12 - prompt_len)
    m.engine.cache.check()
    assert m.engine.cache.num_free(0) == m.engine.cache.num_pages


def test_an_error_inside_a_step_leaves_no_request_open(short_context_dir):
    m = host_model(short_context_dir)
    real_step = m.engine.step
    calls = {"n": 0}

    def failing_step(*a, **kw):
        calls["n"] += 1
        if calls["n"] == 3:
            raise RuntimeError("made-up failure of a step")
        return real_step(*a, **kw)
    m.engine.step = failing_step
    with pytest.raises(RuntimeError, match="made-up failure"):
        m.generate([1, 2, 3], max_tokens=8)
    m.engine.step = real_step
    m.engine.cache.check()
    assert m.engine.cache.num_free(0) == m.engine.cache.num_pages
    assert len(m.generate([1, 2, 3], max_tokens=4)) == 4        # the name "generate" is free again


class _OpsWithAFailedWait(TorchOps):
    """The host backend with the kernel library's error words, one of which is set."""

    def __init__(self):
        self.word = 0
        self.checks = 0

    def check_device_errors(self):
        self.checks += 1
        word, self.word = self.word, 0
        raise_device_errors([("tensor-core GEMM (gemm_tcgen05.cu)", word, {3: "epilogue: the accumulator never arrived"}),
                             ("TMA decode attention (attention_decode_tma.cu)", 0, {})])


def test_a_wait_that_ran_out_is_reported_by_generate_and_by_the_scheduler(short_context_dir):
    ops = _OpsWithAFailedWait()
    cfg = EngineConfig(dtype="float32", page_size=4, num_pages=64, max_batch=2, device="cpu", cuda_graphs=False)
    m = Model(short_context_dir, cfg, ops=ops)
    assert len(m.generate([5, 6], max_tokens=3)) == 3 and ops.checks >= 1
    ops.word = (3 << 16) | 41
    with pytest.raises(KernelError) as e:
        m.generate([5, 6], max_tokens=3)
    text = str(e.value)
    assert "gemm_tcgen05.cu" in text and "block 41" in text and "accumulator never arrived" in text
    assert "attention_decode_tma" not in text
    m.engine.cache.check()
    assert m.engine.cache.num_free(0) == m.engine.cache.num_pages
    ops.word = (3 << 16) | 2
    with pytest.raises(KernelError, match="block 2"):
        m.generate([5, 6], max_tokens=2, use_cache=False)
    assert m.generate([5, 6], max_tokens=2) == m.generate([5, 6], max_tokens=2, use_cache=False)


def test_error_words_are_decoded():
    raise_device_errors([("a", 0, {}), ("b", 0, {})])
    with pytest.raises(KernelError) as e:
        raise_device_errors([("kernel one", (2 << 16) | 7, {2: "copy warp"}), ("kernel two", -1, {}),
                             ("kernel three", (9 << 16) | 1, {})])
    assert "kernel one: a bounded wait ran out in block 7 (copy warp)" in str(e.value)
    assert "kernel two: the error word could not be read" in str(e.value)
    assert "code 9" in str(e.value)


@pytest.mark.parametrize("tied", [False, True])
def test_weight_bytes_count_every_tensor_of_the_file_once(tmp_path, tied):
    """(actual, 32-bit) as the reference reports them (cpp/src/model.cpp:298-318); a tied head is one tensor."""
    import math
    from nanoinfer_b200.weights.safetensors_io import open_model_files
    config = config_from_json_dict(dict(TINY_A, tie_word_embeddings=tied))
    write_random_model(config, str(tmp_path), seed=3)
    shapes = [f.shape(n) for f in open_model_files(str(tmp_path)) for n in f.names()]
    elements = sum(math.prod(s) for s in shapes)
    assert sum(s == (config.vocab_size, config.hidden_size) for s in shapes) == (1 if tied else 2)
    m = host_model(str(tmp_path))
    actual, as_fp32 = m.weight_bytes()
    assert actual == as_fp32 == 4 * elements                   # the host model of the tests is 32-bit throughout
    assert list(m.weight_breakdown()) == ["float32"] and m.weight_breakdown()["float32"][1] == actual
