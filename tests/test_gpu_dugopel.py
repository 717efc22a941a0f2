"""Dugopel through the engine against the plain implementation: each mechanism alone, prompts against
token-by-token decoding, portions, batches, slots and pages used again, far keys and page borders, the first
tokens, long decoding, generation, the two programs, and the kernels alone."""
import numpy as np
import pytest
import torch

import plain_dugopel as plain
import tiny
import tiny_dugopel as td

pytestmark = pytest.mark.gpu

_DIRS, _MODELS = {}, {}


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    def get(name):
        if name not in _DIRS:
            _DIRS[name] = td.write_model(name, tmp_path_factory.mktemp(f"dugopel_{name}"))
        return _DIRS[name]
    return get


@pytest.fixture(scope="module")
def model(folder):
    def get(name, dtype, max_tokens=4096, page_size=16, **kw):
        key = (name, dtype, max_tokens, page_size, tuple(sorted(kw.items())))
        if key not in _MODELS:
            from garlic_inference_b200 import AutoModel
            _MODELS[key] = AutoModel.from_pretrained(folder(name), device=0, dtype=dtype, max_tokens=max_tokens,
                                                     page_size=page_size, **kw)
        return _MODELS[key]
    return get


def _requests(name, lengths, seed):
    return tiny.random_requests(td.TINY[name]["vocab"], lengths, seed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["latent", "dense", "moe", "mix", "wide", "ones"])
def test_prompts_decoding_portions_and_batches_agree_with_the_plain_model(name, dtype, model, folder):
    """Every way of cutting the same requests gives the plain logits: whole prompts; all but 40 tokens, then one
    at a time; portions of 2, 7, 33 and 3 tokens; portions with all requests in one batch; unequal requests that
    start together and decode together.  The cache has room for one batch only, so slots and pages are given back
    and used again by later requests."""
    m = model(name, dtype, max_tokens=512, page_size=16, max_slots=4)
    reqs = _requests(name, [70, 1, 37, 150], seed=5)
    want, own = td.plain_pair(folder(name), reqs)
    for what, steps in (("whole", tiny.trace_whole(reqs)),
                        ("tail", tiny.trace_tail_by_one(reqs, tail=40)),
                        ("portions", td.trace_portions(reqs, [2, 7, 33, 3])),
                        ("portions together", td.trace_portions(reqs, [5, 2, 64], together=True)),
                        ("batched", tiny.trace_batched(reqs, [["r3", "r1"], ["r0", "r2", "r1"]], prompt_frac=0.6))):
        got = tiny.run_trace_in_process(m, steps)
        tiny.assert_covers(got, reqs)
        td.judge(got, want, own, dtype, f"{name} {dtype} {what}")
    assert m.engine.cache.slots.n_free == 4, "every slot came back"
