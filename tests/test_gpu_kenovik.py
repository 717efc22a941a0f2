"""Kenovik through the engine against the plain implementation: each mechanism alone, prompts against
token-by-token decoding, portions, batches, slots and pages used again, far keys at page borders and at the edges
of the distance buckets, the first tokens, long decoding, generation, the two programs, and the kernels alone."""
import math

import numpy as np
import pytest
import torch

import plain_kenovik as plain
import tiny
import tiny_kenovik as tk

pytestmark = pytest.mark.gpu

_DIRS, _MODELS = {}, {}


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    def get(name):
        if name not in _DIRS:
            _DIRS[name] = tk.write_model(name, tmp_path_factory.mktemp(f"kenovik_{name}"))
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
    return tiny.random_requests(tk.TINY[name]["vocab"], lengths, seed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["sink", "bias", "rglru", "dense", "moe", "mix", "tc", "odd", "ones"])
def test_prompts_decoding_portions_and_batches_agree_with_the_plain_model(name, dtype, model, folder):
    """Every way of cutting the same requests gives the plain logits: whole prompts; all but 40 tokens, then one
    at a time; portions of 2, 7, 33 and 3 tokens; portions with all requests in one batch; unequal requests that
    start together and decode together.  The cache has room for one batch only, so slots, pages and state rows are
    given back and used again by later requests."""
    m = model(name, dtype, max_tokens=512, page_size=16, max_slots=4)
    reqs = _requests(name, [70, 1, 37, 150], seed=5)
    want, own = tk.plain_pair(folder(name), reqs)
    for what, steps in (("whole", tiny.trace_whole(reqs)),
                        ("tail", tiny.trace_tail_by_one(reqs, tail=40)),
                        ("portions", tk.trace_portions(reqs, [2, 7, 33, 3])),
                        ("portions together", tk.trace_portions(reqs, [5, 2, 64], together=True)),
                        ("batched", tiny.trace_batched(reqs, [["r3", "r1"], ["r0", "r2", "r1"]], prompt_frac=0.6))):
        got = tiny.run_trace_in_process(m, steps)
        tiny.assert_covers(got, reqs)
        tk.judge_routed(got, want, own, dtype, f"{name} {dtype} {what}", folder(name), reqs)
    assert m.engine.cache.slots.n_free == 4, "every slot came back"


def test_tensor_core_kernels_on_pages_of_64(model, folder):
    """The same on pages of 64 tokens, where prompts of the layers with tensor-core head sizes run the flash kernel
    and their decode steps the split-KV kernel, with the sink and the distance bias inside them."""
    m = model("tc", "bfloat16", max_tokens=2048, page_size=64, max_slots=4)
    reqs = _requests("tc", [200, 3, 129, 64], seed=15)
    want, own = tk.plain_pair(folder("tc"), reqs)
    for steps in (tiny.trace_whole(reqs), tiny.trace_tail_by_one(reqs, tail=70), tk.trace_portions(reqs, [65, 2, 30]),
                  tiny.trace_batched(reqs, [list(reqs)], prompt_frac=0.5)):
        got = tiny.run_trace_in_process(m, steps)
        tiny.assert_covers(got, reqs)
        tk.judge_routed(got, want, own, "bfloat16", "tc on pages of 64", folder("tc"), reqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_of_a_thousand_tokens_through_the_trace_program(dtype, folder, tmp_path):
    """Requests of 1,100, 425, 97 and 1 tokens through bin/trace_run on its default pages of 64: whole, and started
    together with their last 40 % decoded together.  Far keys among a thousand, distances beyond every bias table, the
    query's factor after eight steps, a state carried a thousand tokens."""
    reqs = _requests("long", [1100, 425, 97, 1], seed=17)
    want, own = tk.plain_pair(folder("long"), reqs)
    steps = tiny.trace_whole(reqs) + [dict(s, step=s["step"] + 4, entries=[dict(e, id=e["id"] + "b") for e in s["entries"]],
                                           end=[r + "b" for r in s["end"]])
                                      for s in tiny.trace_batched(reqs, [list(reqs)], prompt_frac=0.6)]
    got = tiny.run_trace_program(folder("long"), dtype, steps, tmp_path / "out", 2048, tk.TINY["long"]["vocab"])
    first = {rid: rows for rid, rows in got.items() if not rid.endswith("b")}
    second = {rid[:-1]: rows for rid, rows in got.items() if rid.endswith("b")}
    for part, what in ((first, "whole"), (second, "together")):
        tiny.assert_covers(part, reqs)
        tk.judge_routed(part, want, own, dtype, f"long {dtype} {what}", folder("long"), reqs)


def test_float32_logits_do_not_depend_on_the_cut_or_the_batch(model):
    """Without routed experts (whose few-row and many-row paths sum in different orders) the same position gives
    the same bits whole, in portions, decoded, alone or in a batch: attention in the exact-order kernel, the
    recurrence walked token by token from the slot's state, every product with a fixed order of sums."""
    for name in ("sink", "bias", "rglru", "dense"):
        m = model(name, "float32", max_tokens=1024, page_size=16)
        reqs = _requests(name, [90, 33], seed=6)
        base = tiny.run_trace_in_process(m, tiny.trace_whole(reqs))
        for steps in (tk.trace_portions(reqs, [2, 31, 8]), tiny.trace_tail_by_one(reqs, tail=20),
                      tk.trace_portions(reqs, [16, 3], together=True)):
            got = tiny.run_trace_in_process(m, steps)
            for rid in reqs:
                for p in range(len(reqs[rid])):
                    assert np.array_equal(got[rid][p], base[rid][p]), f"{name}: request {rid} position {p} differs in its bits"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mix", "tc"])
def test_long_decoding(name, dtype, model, folder):
    """300 tokens decoded one at a time after a prompt of 5, two requests together, through the recorded decode
    step: cache pages taken one by one, distances that pass every bucket's edge and the table's reach, the
    query's factor stepping up, the recurrent state carried 300 times."""
    m = model(name, dtype, max_tokens=1024, page_size=16)
    reqs = _requests(name, [305, 280], seed=9)
    want, own = tk.plain_pair(folder(name), reqs)
    steps = tiny.trace_batched(reqs, [["r0", "r1"]], prompt_frac=5 / 305)
    got = tiny.run_trace_in_process(m, steps)
    tiny.assert_covers(got, reqs)
    tk.judge_routed(got, want, own, dtype, f"long decoding {name} {dtype}", folder(name), reqs)
    assert m.engine.graphs is not None and 2 in m.engine.graphs._graphs, "decode steps ran from a recorded graph"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["moe", "mix", "tc"])
def test_a_dozen_requests_decode_together(name, dtype, model, folder):
    """Twelve unequal requests start together and decode together through a recorded step of 16 rows (four of them
    padding): the routed feed-forward runs expert by expert inside the recording, the kernels see padding rows
    (slot -1: no state, no page), and requests leave one after the other."""
    m = model(name, dtype, max_tokens=2048, page_size=16, max_slots=12)
    reqs = _requests(name, [31 + 3 * i for i in range(12)], seed=21)
    want, own = tk.plain_pair(folder(name), reqs)
    got = tiny.run_trace_in_process(m, tiny.trace_batched(reqs, [list(reqs)], prompt_frac=0.5))
    tiny.assert_covers(got, reqs)
    tk.judge_routed(got, want, own, dtype, f"twelve together {name} {dtype}", folder(name), reqs)
    assert m.engine.graphs is not None and 16 in m.engine.graphs._graphs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(dtype, model, folder):
    m = model("mix", dtype, max_tokens=512, page_size=16, max_slots=3)
    prompts = list(_requests("mix", [9, 1, 30, 17, 5], seed=10).values())
    got = m.generate(prompts, max_new_tokens=10)
    assert m.last_stats.batches == 2
    cfg, w = plain.read_model_dir(folder("mix"))
    for prompt, new in zip(prompts, got):
        ids = list(prompt)
        assert len(new) == 10
        for k, tok in enumerate(new):
            logits = plain.forward(cfg, w, ids)[-1]
            best = int(logits.argmax())
            if tok != best:
                gap = float(logits[best] - logits[tok]) / float(logits.abs().max())
                assert dtype == "bfloat16" and gap <= 0.1, \
                    f"prompt of {len(prompt)}, new token {k}: engine chose {tok}, plain {best} (gap {gap:.2e})"
                break
            ids.append(tok)


def test_trace_program_and_command_line_serve_the_design(folder, tmp_path):
    import subprocess
    import sys
    reqs = _requests("odd", [20, 3], seed=12)
    want, own = tk.plain_pair(folder("odd"), reqs)
    steps = tiny.trace_batched(reqs, [["r0", "r1"]])
    got = tiny.run_trace_program(folder("odd"), "float32", steps, tmp_path / "out", 256, tk.TINY["odd"]["vocab"])
    tk.judge(got, want, own, "float32", "trace program")
    r = subprocess.run([sys.executable, str(tiny.REPO / "bin" / "runner"), str(folder("odd")), "--prompt-ids", "5,6,7",
                        "--max-new-tokens", "4", "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    ids = [int(t) for t in r.stdout.splitlines()[0].split()]
    cfg, w = plain.read_model_dir(folder("odd"))
    seq = [5, 6, 7]
    for tok in ids:
        assert tok == int(plain.forward(cfg, w, seq)[-1].argmax())
        seq.append(tok)


def test_a_folder_without_the_bias_table_row_count_in_its_config(folder, tmp_path):
    """The number of distance buckets is no key of the design: a folder whose config.json lacks this library's own
    key gets it from the stored table's shape."""
    import json
    from garlic_inference_b200 import AutoModel
    src = folder("bias")
    dst = tmp_path / "bare"
    dst.mkdir()
    cfg = json.loads((src / "config.json").read_text())
    assert cfg["layers"][0]["mixer"].pop("bias_rows") == 10
    (dst / "config.json").write_text(json.dumps(cfg))
    (dst / "model.safetensors").symlink_to(src / "model.safetensors")
    m = AutoModel.from_pretrained(dst, device=0, dtype="float32", max_tokens=256, page_size=16)
    reqs = _requests("bias", [60], seed=2)
    want, own = tk.plain_pair(dst, reqs)
    tk.judge(tiny.run_trace_in_process(m, tiny.trace_whole(reqs)), want, own, "float32", "rows from the tensor")


# ---- kernels alone -----------------------------------------------------------------------------
def _paged(keys, values, page, spare=3):
    """Pools and a block table (slot 1) that hold keys [T, G, d] and values [T, G, dv] on pages out of order."""
    T, G, d = keys.shape
    dv = values.shape[2]
    n_pages = -(-T // page)
    order = torch.randperm(n_pages + spare)[:n_pages]
    k_pool = torch.zeros(n_pages + spare, G, page, d, dtype=keys.dtype, device="cuda")
    v_pool = torch.zeros(n_pages + spare, G, page, dv, dtype=keys.dtype, device="cuda")
    for j in range(T):
        k_pool[order[j // page], :, j % page] = keys[j]
        v_pool[order[j // page], :, j % page] = values[j]
    table = torch.full((2, n_pages + 1), -1, dtype=torch.int32, device="cuda")
    table[1, :n_pages] = order.to(torch.int32)
    return k_pool, v_pool, table


def _plain_attention(q, k, v, scale, sink, table_by_distance):
    """o[t, h] over keys j <= t; `sink` a score in the denominator or None; table_by_distance [>= T, H] or None."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=torch.float64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h].double() @ k[:, g].double().T) * scale
        if table_by_distance is not None:
            dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).clamp(min=0)
            s = s + table_by_distance[:, h].double()[dist]
        s = torch.where(torch.arange(T)[None, :] <= torch.arange(T)[:, None], s, torch.full_like(s, -math.inf))
        if sink is not None:
            s0 = float(sink[h]) if isinstance(sink, (list, tuple)) else float(sink)
            s = torch.cat([s, torch.full((T, 1), s0, dtype=torch.float64)], 1)
        p = torch.softmax(s, -1)[:, :T]
        out[:, h] = p @ v[:, g].double()
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_a_sink_and_a_far_key_that_stands_out(dtype):
    """One key is made several times as large as the others and the queries are given a part along it, so nearly
    all the weight of every later query lies on that key, wherever it sits: position 0, a page's last row, the next
    page's first, hundreds of keys back.  Then the same with every score far below the sink's, where the output all
    but vanishes.  Exact-order kernel, flash kernel for prompts, split-KV kernel for single tokens."""
    from garlic_inference_b200.ops import kernels
    from garlic_inference_b200.parts import StepShape
    from garlic_inference_b200.parts.attention import query_runs
    torch.manual_seed(4)
    H, G, d, dv, page, T, scale = 6, 2, 32, 64, 16, 300, 0.3
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    slot = torch.ones(T, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    sinks = torch.zeros(H, device="cuda")
    runs = torch.from_numpy(query_runs(StepShape([1], [0], [T], [0], False), 64)).cuda()
    for far, boost in ((0, 1.0), (15, 1.0), (16, 1.0), (17, 1.0), (63, 1.0), (64, 1.0), (130, 1.0), (40, -1.0)):
        k = torch.randn(T, G, d) * 0.3
        v = torch.randn(T, G, dv)
        q = torch.randn(T, H, d) * 0.3
        k[far, :, :8] = 6.0
        q[:, :, :8] = 1.5 * boost                     # boost -1: every query is pushed away from that key
        if boost < 0:
            k[:, :, :8] = 6.0                         # ... and from every other key: all scores far below the sink's 0
        q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
        want = _plain_attention(q.float(), k.float(), v.float(), scale, 0.0, None)
        if boost > 0:
            late = want[max(far, 200):] - v[far].float().repeat_interleave(H // G, 0).double()
            assert float(late.abs().max()) < 1e-2, "nearly all the weight is on the far key"
        else:
            assert float(want.abs().max()) < 1e-3, "the sink takes nearly all the weight"
        if far != 0:
            without = _plain_attention(q.float(), k.float(), v.float(), scale, None, None)
            assert float((without - want)[0].abs().max()) > 0.05, "the sink shows at the first token"
        k_pool, v_pool, table = _paged(k.cuda(), v.cuda(), page)
        got = kernels.attention_masked(q.cuda(), k_pool, v_pool, table, pos, slot, scale, status, sinks=sinks, out_float32=True)
        torch.testing.assert_close(got.cpu().double().view(T, H, dv), want, **tol)
        if dtype == torch.bfloat16:
            got = kernels.attention_prefill_masked_bf16(q.cuda(), k_pool, v_pool, table, runs, scale, sinks=sinks,
                                                        rows_covered=True)
            torch.testing.assert_close(got.cpu().double().view(T, H, dv), want, **tol)
            last = torch.tensor([T - 1, 201, far, 0], device="cuda")
            for n_splits in (1, 3):
                one = kernels.attention_decode_masked_bf16(q.cuda()[last].contiguous(), k_pool, v_pool, table,
                                                           pos[last].contiguous(), slot[last].contiguous(), scale,
                                                           n_splits=n_splits, sinks=sinks)
                torch.testing.assert_close(one.cpu().double().view(4, H, dv), want[last.cpu()], **tol)
    assert int(status.item()) == 0


def test_tcgen05_prompt_attention_with_sinks():
    """The tcgen05 flash kernel (heads of 128, pages of 64) with a sink per head, among them one far above every score
    and one far below: rows of three sequences, one of them continuing from cached keys."""
    from garlic_inference_b200.ops import kernels
    from garlic_inference_b200.parts import StepShape
    from garlic_inference_b200.parts.attention import query_runs
    torch.manual_seed(10)
    H, G, d, page, T, scale = 4, 2, 128, 64, 333, 0.1
    sink = [0.0, 30.0, -40.0, 1.5]
    k, v, q = torch.randn(T, G, d).bfloat16(), torch.randn(T, G, d).bfloat16(), torch.randn(T, H, d).bfloat16()
    want = _plain_attention(q.float(), k.float(), v.float(), scale, sink, None)
    assert float(want[:, 1].abs().max()) < 1e-6 and float(want[0, 2].double().sub(v[0, 1].double()).abs().max()) < 1e-6
    k_pool, v_pool, table = _paged(k.cuda(), v.cuda(), page)
    # the last 133 rows as a step that continues a sequence of 200 cached tokens, runs of 128
    runs = torch.from_numpy(query_runs(StepShape([1], [0], [133], [200], False), 128)).cuda()
    got = kernels.attention_prefill_tcgen05(q[200:].contiguous().cuda(), k_pool, v_pool, table, runs, scale, 0, rows_covered=True,
                                            sinks=torch.tensor(sink, device="cuda"))
    torch.testing.assert_close(got.cpu().double().view(133, H, d), want[200:], rtol=3e-2, atol=3e-2)
    kernels.check_bounded_waits(torch.device("cuda", 0))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_a_distance_bias_whose_one_bucket_stands_out(dtype):
    """The bias table is large in one row and zero elsewhere, and queries and keys are small: every query then reads
    the mean of the values whose distance falls into that row's bucket, so a bucket's edge that is one distance off
    moves the result by a whole value.  Rows: one of the exact distances, the first logarithmic bucket, one in the
    middle, the last (which also takes every distance from the table's reach on)."""
    from garlic_inference_b200.ops import kernels
    from garlic_inference_b200.parts import MaskedAttention, StepShape
    from garlic_inference_b200.parts.attention import query_runs
    torch.manual_seed(5)
    H, G, d, dv, page, T, scale, rows, reach = 4, 2, 64, 32, 16, 260, 0.2, 12, 90
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    slot = torch.ones(T, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    runs = torch.from_numpy(query_runs(StepShape([1], [0], [T], [0], False), 64)).cuda()
    buckets = MaskedAttention.distance_buckets(rows, reach)
    assert buckets.tolist() == [plain.distance_bucket(n, rows, reach) for n in range(reach + 1)]
    for row in (3, 6, 9, 11):
        rel = torch.zeros(rows, H)
        rel[row] = torch.tensor([14.0, 15.0, 16.0, 17.0])
        by_distance = rel[torch.tensor([plain.distance_bucket(n, rows, reach) for n in range(T)])]      # [T, H]
        k = torch.randn(T, G, d) * 0.05
        v = torch.randn(T, G, dv)
        q = torch.randn(T, H, d) * 0.05
        q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
        want = _plain_attention(q.float(), k.float(), v.float(), scale, None, by_distance)
        inside = [n for n in range(T) if plain.distance_bucket(n, rows, reach) == row]
        t = T - 1
        mean = torch.stack([v[t - n].float() for n in inside]).mean(0).repeat_interleave(H // G, 0)
        assert float((want[t] - mean.double()).abs().max()) < 0.05, "the last query reads its bucket's values"
        table_dev = rel[buckets].contiguous().cuda()           # what the mixer hands to the kernels: [reach + 1, H]
        k_pool, v_pool, table = _paged(k.cuda(), v.cuda(), page)
        got = kernels.attention_masked(q.cuda(), k_pool, v_pool, table, pos, slot, scale, status, dist_bias=table_dev,
                                       out_float32=True)
        torch.testing.assert_close(got.cpu().double().view(T, H, dv), want, **tol)
        if dtype == torch.bfloat16:
            got = kernels.attention_prefill_masked_bf16(q.cuda(), k_pool, v_pool, table, runs, scale, dist_bias=table_dev,
                                                        rows_covered=True)
            torch.testing.assert_close(got.cpu().double().view(T, H, dv), want, **tol)
            last = torch.tensor([T - 1, 100, reach, reach - 1, 5, 0], device="cuda")
            one = kernels.attention_decode_masked_bf16(q.cuda()[last].contiguous(), k_pool, v_pool, table,
                                                       pos[last].contiguous(), slot[last].contiguous(), scale,
                                                       n_splits=2, dist_bias=table_dev)
            torch.testing.assert_close(one.cpu().double().view(len(last), H, dv), want[last.cpu()], **tol)
    assert int(status.item()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_queries_and_cache_rows_with_bias_projection_norm_temperature_and_scaled_rotation(dtype):
    """The kernel between projections and attention: biases, the RMS norm over all of a token's query (and key)
    columns at once, the factor that grows with the position (steps at positions every - 1, 2 every - 1, ...), the
    rotation of pairs with divided frequencies, keys and values into pages out of order."""
    from garlic_inference_b200.ops import kernels
    torch.manual_seed(6)
    H, G, d, dv, page, T = 3, 1, 10, 6, 16, 70
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    cols = H * d + G * d + G * dv
    src = torch.randn(T, cols + 9, device="cuda").to(dtype)[:, 9:]
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    slot = torch.ones(T, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = src.float().cpu()
    xq, xk, xv = x[:, :H * d], x[:, H * d:H * d + G * d], x[:, H * d + G * d:]

    def cached(pool, table, width):
        n_pages = table.shape[1] - 1
        return pool[table[1, :n_pages].long()].permute(0, 2, 1, 3).reshape(-1, pool.shape[1], width)[:T].float().cpu()

    # biases and a rotation of 6 of 10 dimensions with frequencies divided by 4
    bias = torch.randn(cols, device="cuda")
    freq = torch.tensor([50.0 ** (-2.0 * i / 6) / 4.0 for i in range(3)], dtype=torch.float32, device="cuda")
    k_pool, v_pool, table = _paged(torch.zeros(T, G, d, device="cuda", dtype=dtype), torch.zeros(T, G, dv, device="cuda", dtype=dtype), page)
    q = kernels.attn_prepare(src, 0, H * d, H * d + G * d, freq, 6, False, pos, slot, table, k_pool, v_pool, H, d, dtype,
                             status, bias=bias)
    b = bias.cpu()
    want_q = plain.rotate_pairs((xq + b[:H * d]).view(T, H, d), torch.arange(T), 6, 50.0, 4.0)
    want_k = plain.rotate_pairs((xk + b[H * d:H * d + G * d]).view(T, G, d), torch.arange(T), 6, 50.0, 4.0)
    torch.testing.assert_close(q.float().cpu(), want_q, **tol)
    torch.testing.assert_close(cached(k_pool, table, d), want_k, **tol)
    torch.testing.assert_close(cached(v_pool, table, dv), (xv + b[H * d + G * d:]).view(T, G, dv), **tol)
    # the norm over the whole projection and the query's factor, no rotation
    wn = (1 + 0.3 * torch.randn(H * d + G * d)).cuda()
    k_pool, v_pool, table = _paged(torch.zeros(T, G, d, device="cuda", dtype=dtype), torch.zeros(T, G, dv, device="cuda", dtype=dtype), page)
    q = kernels.attn_prepare(src, 0, H * d, H * d + G * d, None, 0, False, pos, slot, table, k_pool, v_pool, H, d, dtype,
                             status, norm_weight=wn, norm_eps=1e-3, temp_coef=0.7, temp_every=16)
    temp = plain.query_temperature(torch.arange(T), 0.7, 16, torch.float32)
    assert float(temp[14]) == 1.0 and float(temp[15]) > 1.4 and float(temp[30]) == float(temp[15]) < float(temp[31])
    want_q = plain.rms_norm(xq, wn.cpu()[:H * d], 1e-3) * temp[:, None]
    torch.testing.assert_close(q.float().cpu().view(T, H * d), want_q, **tol)
    torch.testing.assert_close(cached(k_pool, table, d).view(T, G * d), plain.rms_norm(xk, wn.cpu()[H * d:], 1e-3), **tol)
    torch.testing.assert_close(cached(v_pool, table, dv).view(T, G * dv), xv, **tol)
    assert int(status.item()) == 0


def test_router_with_sigmoid_scores_a_correction_and_groups_judged_by_their_two_best():
    from garlic_inference_b200.ops import kernels
    torch.manual_seed(7)
    for n, E, top, groups, keep, scale in ((45, 12, 5, 4, 2, 2.5), (7, 6, 3, 3, 2, 1.0), (300, 64, 6, 8, 3, 0.5),
                                           (5, 1, 1, 1, 1, 1.0), (9, 40, 40, 5, 5, 1.0), (11, 8, 2, 8, 4, 3.0)):
        z = torch.randn(n, E, device="cuda") * 2
        corr = torch.randn(E, device="cuda")
        router = {"experts": E, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}
        idx, wt = kernels.router_select(z, top, groups, keep, scale, sigmoid=True, correction=corr, group_top=2, normalize=True)
        ri, rw = plain.route(z.cpu(), {"router": torch.eye(E), "correction": corr.cpu()}, router)
        assert torch.equal(idx.cpu().long(), ri), f"{E} experts, {groups} groups"
        torch.testing.assert_close(wt.cpu(), rw, rtol=1e-5, atol=1e-7)
    # group scores by the two best: group 0 holds the single best expert, group 1 the better pair; only one group stays.
    # The correction turns the choice without touching the weights, and can make choosing scores negative.
    s = torch.tensor([[0.9, 0.1, 0.6, 0.55]])
    z = torch.log(s / (1 - s)).cuda()
    zero = torch.zeros(4, device="cuda")
    idx, wt = kernels.router_select(z, 1, 2, 1, 2.0, sigmoid=True, correction=zero, group_top=2, normalize=True)
    assert idx.tolist() == [[2]] and torch.allclose(wt.cpu(), torch.tensor([[2.0]]))
    idx, _ = kernels.router_select(z, 1, 2, 1, 2.0, sigmoid=True, correction=zero, group_top=1, normalize=True)
    assert idx.tolist() == [[0]]
    corr = torch.tensor([-3.0, -3.2, -9.0, -9.0], device="cuda")
    idx, wt = kernels.router_select(z, 2, 2, 1, 1.0, sigmoid=True, correction=corr, group_top=2, normalize=True)
    assert idx.tolist() == [[0, 1]] and torch.allclose(wt.cpu(), torch.tensor([[0.9, 0.1]]), atol=1e-6)


def test_recurrent_unit_gates_scan_and_convolution_with_biases():
    """The three kernels of the recurrent block against the plain functions, a prompt cut into steps of 1, 2, 9 and
    the rest with the state carried in a slot's row, beside a second sequence and a padding row."""
    from garlic_inference_b200.ops import kernels
    torch.manual_seed(8)
    for W, B, K in ((60, 5, 4), (48, 1, 1), (33, 3, 2), (256, 2, 3), (2048, 2, 2)):      # the last: blocks too wide for shared memory
        bw, T = W // B, 41
        m = {"width": W, "blocks": B, "conv": K}
        Wt = {"y": torch.zeros(W, 1), "y.b": torch.randn(W), "x": torch.zeros(W, 1), "x.b": torch.randn(W) * 0.3,
              "conv": torch.randn(W, K) * 0.6, "conv.b": torch.randn(W) * 0.2, "ra": torch.randn(B, bw, bw) * 0.4,
              "ra.b": torch.randn(B, bw), "ri": torch.randn(B, bw, bw) * 0.4, "ri.b": torch.randn(B, bw),
              "lam": torch.randn(W) * 2, "o": torch.eye(W)}
        xin, yin = torch.randn(T, W), torch.randn(T, W)
        Wp = dict(Wt)
        # the plain block with the two projections' results given: h = [yin | xin], picked by identity-like matrices
        h = torch.cat([yin, xin], 1)
        Wp["y"] = torch.cat([torch.eye(W), torch.zeros(W, W)], 1)
        Wp["x"] = torch.cat([torch.zeros(W, W), torch.eye(W)], 1)
        want = plain.rglru(h.double(), {k: v.double() for k, v in Wp.items()}, m)
        dev = {k: v.cuda() for k, v in Wt.items()}
        state = torch.zeros(4, (K * W + 3) // 4 * 4, device="cuda")
        other = torch.randn(3, 2 * W, device="cuda")
        got = []
        at = 0
        for n in (1, 2, 9, T - 12):
            # rows: the other sequence's (slot 0), then this one's n rows (slot 2), then a padding row
            proj = torch.cat([other, h[at:at + n].cuda(), torch.zeros(1, 2 * W, device="cuda")])
            slots = torch.tensor([0] * 3 + [2] * n + [-1], dtype=torch.int32, device="cuda")
            spans = torch.tensor([[2, 3, n], [0, 0, 3], [-1, 3 + n, 1]], dtype=torch.int32, device="cuda")
            conv_state = state[:, W:] if K > 1 else state
            u = kernels.causal_conv_silu(proj[:, W:], dev["conv"], conv_state, slots, activation="none",
                                         in_bias=dev["x.b"], out_bias=dev["conv.b"])
            kernels.conv_state_update(proj[:, W:], K, conv_state, slots, in_bias=dev["x.b"])
            a, b = kernels.rglru_gates(u, dev["ra"].transpose(1, 2).contiguous(), dev["ri"].transpose(1, 2).contiguous(),
                                       dev["ra.b"].reshape(-1), dev["ri.b"].reshape(-1), dev["lam"], 8.0)
            assert float(a.min()) >= 0.0 and float(a.max()) <= 1.0
            out = kernels.rglru_scan(a, b, proj[:, :W], dev["y.b"], state, spans, slots)
            got.append(out[3:3 + n].cpu())
            assert float(out[-1].abs().max()) == 0.0, "a padding row gives zeros"
            at += n
        torch.testing.assert_close(torch.cat(got).double(), want, rtol=2e-4, atol=2e-5)
        assert float(state[3].abs().max()) == 0.0 and float(state[1].abs().max()) == 0.0, "no other slot's row was touched"


def test_norm_takes_a_vector_along_and_the_weighted_sum_an_addend():
    from garlic_inference_b200.ops import kernels
    torch.manual_seed(9)
    for dim in (100, 48, 2050):
        res = torch.randn(37, dim, device="cuda") * 3
        d1, w, off = torch.randn(37, dim, device="cuda"), torch.randn(dim, device="cuda"), torch.randn(dim, device="cuda")
        keep = res.clone()
        out = kernels.add_rmsnorm(d1, res, w, 1e-5, torch.float32, offset=off)
        s = keep.cpu() + d1.cpu() + off.cpu()
        torch.testing.assert_close(res.cpu(), s, rtol=1e-6, atol=1e-6)
        torch.testing.assert_close(out.cpu(), plain.rms_norm(s, w.cpu(), 1e-5), rtol=1e-5, atol=1e-5)
        only = kernels.add_rmsnorm(None, keep.clone(), w, 1e-5, torch.float32, offset=off)
        torch.testing.assert_close(only.cpu(), plain.rms_norm(keep.cpu() + off.cpu(), w.cpu(), 1e-5), rtol=1e-5, atol=1e-5)
        again = keep.clone()
        kernels.residual_add_row(off, again)
        torch.testing.assert_close(again.cpu(), keep.cpu() + off.cpu(), rtol=1e-6, atol=1e-6)
    buf, wt, add = torch.randn(12, 40, device="cuda"), torch.rand(4, 3, device="cuda"), torch.randn(4, 40, device="cuda")
    got = kernels.moe_combine(buf, None, wt, add)
    want = add.cpu() + (buf.cpu().view(4, 3, 40) * wt.cpu()[:, :, None]).sum(1)
    torch.testing.assert_close(got.cpu(), want, rtol=1e-5, atol=1e-6)


def test_routed_experts_with_a_shared_expert_few_rows_and_many_rows_agree(folder):
    """The part's two ways (row by row for a few tokens, expert by expert for many) on the same rows, and both
    against the plain feed-forward."""
    from garlic_inference_b200.parts import Runtime, StepContext, part_class
    from garlic_inference_b200.weights import Checkpoint
    ck = Checkpoint(folder("moe"))
    spec = tk.make_config("moe").plan().layers[0].feed_forward

    class Load:
        def dtype(self, *a):
            return torch.float32

        def __call__(self, n, out=None):
            t = ck.tensor(spec.weights[n]).float().cuda()
            return t if out is None else out.copy_(t)

    part = part_class("routed_experts")(spec.params, Load(), Runtime(torch.float32, torch.device("cuda")))
    x = torch.randn(70, 48, device="cuda")
    z = torch.zeros(70, dtype=torch.int32, device="cuda")
    many = part.step(x, StepContext(70, z, z, z))
    few = torch.cat([part.step(x[i:i + 7].contiguous(), StepContext(7, z, z, z)) for i in range(0, 70, 7)])
    torch.testing.assert_close(many, few, rtol=1e-5, atol=1e-6)
    w = {n[len("l0.mlp."):]: ck.tensor(n).float() for n in ck.names() if n.startswith("l0.mlp.")}
    torch.testing.assert_close(many.cpu(), plain.moe_ff(x.cpu(), w, tk.config_dict("moe")["layers"][0]["mlp"]), rtol=1e-4, atol=1e-5)
