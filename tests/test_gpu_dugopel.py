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
@pytest.mark.parametrize("name", ["latent", "dense", "moe", "mix", "wide", "odd", "ones"])
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


def test_float32_logits_do_not_depend_on_the_cut_or_the_batch(model):
    """Without routed experts (whose few-row and many-row paths sum in different orders) the same position gives
    the same bits whole, in portions, decoded, alone or in a batch."""
    for name in ("latent", "dense"):
        m = model(name, "float32", max_tokens=1024, page_size=16)
        reqs = _requests(name, [90, 33], seed=6)
        base = tiny.run_trace_in_process(m, tiny.trace_whole(reqs))
        for steps in (td.trace_portions(reqs, [2, 31, 8]), tiny.trace_tail_by_one(reqs, tail=20),
                      td.trace_portions(reqs, [16, 3], together=True)):
            got = tiny.run_trace_in_process(m, steps)
            for rid in reqs:
                for p in range(len(reqs[rid])):
                    assert np.array_equal(got[rid][p], base[rid][p]), f"{name}: request {rid} position {p} differs in its bits"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_at_page_borders_and_the_first_tokens(dtype, folder, tmp_path):
    """The norms take every token's size away, so a far key is made to stand out through the weights: one channel of
    the embedding is zero for every token but one, and the shared rotated key part reads that channel with large
    factors.  That token stands at positions 0, 15, 16, 17, 63 and 64 (cache pages of 16) of a prompt of 700; its
    rotated key part is several times the others', so queries hundreds of positions later weigh it heavily, with a
    sign that turns with the distance.  The plain model says how much a lost or misplaced key would show (the same
    prompt without those tokens), and the engine has to be far closer than that: whole, with a decoded tail, and in
    portions of 17 and 2."""
    from garlic_inference_b200 import AutoModel
    from garlic_inference_b200.weights.safetensors_io import SafetensorsFile, write_safetensors_lazy
    src = folder("latent")
    f = SafetensorsFile(src / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    needle, rank = 7, td.TINY["latent"]["layers"][0]["mixer"]["kv_rank"]
    tensors["embed"][:, 0] = 0
    tensors["embed"][needle, 0] = 1.0
    tensors["l0.mix.dkv"][rank:, 0] = torch.tensor([1.5, -1.0, 0.5, 2.0, -1.5, 1.0, -0.5, 1.0]).to(tensors["l0.mix.dkv"].dtype)
    dst = tmp_path / "needle"
    dst.mkdir()
    (dst / "config.json").write_text((src / "config.json").read_text())
    write_safetensors_lazy(dst / "model.safetensors", {n: (t.dtype, tuple(t.shape)) for n, t in tensors.items()},
                           lambda n: tensors[n])
    rng = np.random.default_rng(3)
    toks = [int(t) for t in rng.integers(8, 300, size=700)]
    plainer = list(toks)
    for p in (0, 15, 16, 17, 63, 64):
        toks[p] = needle
    ends = (20, 65, 300, 500, 640, 699)
    cfg, w = plain.read_model_dir(dst)
    want = plain.forward(cfg, w, toks, torch.float64).numpy()
    own = plain.forward(cfg, w, toks, torch.float32).double().numpy()
    without = plain.forward(cfg, w, plainer, torch.float64).numpy()
    shows = min(np.sqrt(((want[p] - without[p]) ** 2).mean()) for p in ends) / np.sqrt((want ** 2).mean())
    assert shows > 5 * td.BF16_MEDIAN, f"the far keys move the logits by only {shows:.2e}"
    m = AutoModel.from_pretrained(dst, device=0, dtype=dtype, max_tokens=1024, page_size=16)
    reqs = {"n": toks}
    for steps in (tiny.trace_whole(reqs), tiny.trace_tail_by_one(reqs, tail=62), td.trace_portions(reqs, [17, 2])):
        got = tiny.run_trace_in_process(m, steps)
        td.judge(got, {"n": want}, {"n": own}, dtype, f"far keys {dtype}")
        if dtype == "bfloat16":                   # the rows that look far back, one by one
            errs = td.row_errors(got, {"n": want})
            assert max(errs[("n", p)][1] for p in ends) <= shows / 5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mix", "moe"])
def test_long_decoding(name, dtype, model, folder):
    """300 tokens decoded one at a time after a prompt of 5, two requests together, through the recorded decode
    step: cache pages taken one by one, borrowed rows read in the step that wrote them."""
    m = model(name, dtype, max_tokens=1024, page_size=16)
    reqs = _requests(name, [305, 280], seed=9)
    want, own = td.plain_pair(folder(name), reqs)
    steps = tiny.trace_batched(reqs, [["r0", "r1"]], prompt_frac=5 / 305)
    got = tiny.run_trace_in_process(m, steps)
    tiny.assert_covers(got, reqs)
    td.judge(got, want, own, dtype, f"long decoding {name} {dtype}")
    assert m.engine.graphs is not None and 2 in m.engine.graphs._graphs, "decode steps ran from a recorded graph"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["moe", "mix", "wide", "odd"])
def test_a_dozen_requests_decode_together(name, dtype, model, folder):
    """Twelve unequal requests start together and decode together through a recorded step of 16 rows (four of them
    padding): the routed feed-forward then runs expert by expert inside the recording, the attention kernels see
    padding rows, and requests leave one after the other."""
    m = model(name, dtype, max_tokens=2048, page_size=16, max_slots=12)
    reqs = _requests(name, [31 + 3 * i for i in range(12)], seed=21)
    want, own = td.plain_pair(folder(name), reqs)
    got = tiny.run_trace_in_process(m, tiny.trace_batched(reqs, [list(reqs)], prompt_frac=0.5))
    tiny.assert_covers(got, reqs)
    td.judge(got, want, own, dtype, f"twelve together {name} {dtype}")
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
    reqs = _requests("ones", [20, 3], seed=12)
    want, own = td.plain_pair(folder("ones"), reqs)
    steps = tiny.trace_batched(reqs, [["r0", "r1"]])
    got = tiny.run_trace_program(folder("ones"), "float32", steps, tmp_path / "out", 256, td.TINY["ones"]["vocab"])
    td.judge(got, want, own, "float32", "trace program")
    r = subprocess.run([sys.executable, str(tiny.REPO / "bin" / "runner"), str(folder("ones")), "--prompt-ids", "5,6,7",
                        "--max-new-tokens", "4", "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    ids = [int(t) for t in r.stdout.splitlines()[0].split()]
    cfg, w = plain.read_model_dir(folder("ones"))
    seq = [5, 6, 7]
    for tok in ids:
        assert tok == int(plain.forward(cfg, w, seq)[-1].argmax())
        seq.append(tok)


def test_one_output_product_serves_both_sublayers_of_a_dense_layer(model):
    """A layer with a dense feed-forward joins its two output projections into one product; a routed one leaves two
    pending results for the next norm."""
    m = model("mix", "bfloat16", max_tokens=512, page_size=16, max_slots=3)
    blocks = m.model.blocks
    assert blocks[1].w_out is not None and blocks[1].w_out.shape == (96, 6 * 16 + 128) and blocks[1].mixer.w_o is None
    assert blocks[0].w_out is None and blocks[0].mixer.w_o is not None
    assert blocks[3].feed_forward is None and blocks[3].w_out is None


# ---- kernels alone -----------------------------------------------------------------------------
def test_layer_norm_with_two_pending_results_rms_rows_and_cap():
    from garlic_inference_b200.ops import kernels
    torch.manual_seed(0)
    for dim in (100, 48, 2050):
        res = torch.randn(37, dim, device="cuda") * 3 + 1.5
        d1, d2, w, b = (torch.randn(s, device="cuda") for s in ((37, dim), (37, dim), (dim,), (dim,)))
        keep = res.clone()
        out = kernels.add_layernorm(d1, res, w, None, 1e-5, torch.float32, delta2=d2)
        s = keep.cpu() + (d1.cpu() + d2.cpu())
        torch.testing.assert_close(res.cpu(), s, rtol=1e-6, atol=1e-6)
        torch.testing.assert_close(out.cpu(), plain.layer_norm(s, w.cpu(), 1e-5), rtol=1e-5, atol=1e-5)
        rows = torch.tensor([5, 0, 36], dtype=torch.int32, device="cuda")
        before = res.clone()
        picked = kernels.add_layernorm(d1, res, w, b, 1e-5, torch.float32, rows=rows)
        assert torch.equal(res, before), "gathered rows write nothing back"
        want = plain.layer_norm((before + d1).cpu()[[5, 0, 36]], w.cpu(), 1e-5) + b.cpu()
        torch.testing.assert_close(picked.cpu(), want, rtol=1e-5, atol=1e-5)
        only2 = kernels.add_layernorm(None, keep.clone(), w, None, 1e-5, torch.float32, delta2=d2)
        torch.testing.assert_close(only2.cpu(), plain.layer_norm(keep.cpu() + d2.cpu(), w.cpu(), 1e-5), rtol=1e-5, atol=1e-5)
        few = kernels.add_layernorm(None, res[:3].contiguous(), w.bfloat16(), None, 1e-5, torch.bfloat16)
        torch.testing.assert_close(few.float().cpu(), plain.layer_norm(res[:3].cpu(), w.bfloat16().float().cpu(), 1e-5),
                                   rtol=1e-2, atol=1e-2)
    # a row far from zero with a small spread: the variance comes from the deviations, not from a difference of squares
    res = (100.0 + torch.randn(4, 64)).cuda()
    out = kernels.add_layernorm(None, res, torch.ones(64, device="cuda"), None, 1e-9, torch.float32)
    torch.testing.assert_close(out.cpu(), plain.layer_norm(res.cpu().double(), torch.ones(64, dtype=torch.float64), 1e-9).float(),
                               rtol=1e-3, atol=1e-3)
    wide = torch.randn(9, 70, device="cuda")
    w = torch.randn(24, device="cuda")
    got = kernels.rmsnorm_rows(wide[:, 11:35], w, 1e-6)
    torch.testing.assert_close(got.cpu(), plain.rms_norm(wide[:, 11:35].cpu(), w.cpu(), 1e-6), rtol=1e-5, atol=1e-6)
    z = torch.randn(5, 33, device="cuda") * 40
    torch.testing.assert_close(kernels.softcap_(z.clone(), 12.0).cpu(), 12.0 * torch.tanh(z.cpu() / 12.0), rtol=1e-5, atol=1e-5)


def test_gated_unit_with_limits_and_a_shift():
    from garlic_inference_b200.ops import kernels
    torch.manual_seed(1)
    gu = torch.randn(9, 140, device="cuda") * 3
    g, u = gu[:, :70].cpu(), gu[:, 70:].cpu()
    unit = kernels.glu_shape("swish", 1.702, 1.1, 1.1, 1.0)
    want = torch.clamp(g, max=1.1)
    want = want * plain.sigmoid(1.702 * want) * (torch.clamp(u, -1.1, 1.1) + 1.0)
    torch.testing.assert_close(kernels.glu(gu, unit).cpu(), want, rtol=1e-5, atol=1e-6)
    out = torch.zeros(9, 100, device="cuda")
    kernels.glu(gu, unit, out=out[:, 20:90])
    torch.testing.assert_close(out[:, 20:90].cpu(), want, rtol=1e-5, atol=1e-6)
    assert float(out[:, :20].abs().max()) == 0.0 and float(out[:, 90:].abs().max()) == 0.0
    gb = (torch.randn(5, 64, device="cuda") * 3).bfloat16()          # the 16-byte path
    gf = gb.float().cpu()
    w2 = torch.clamp(gf[:, :32], max=0.5)
    w2 = w2 * plain.sigmoid(1.702 * w2) * (torch.clamp(gf[:, 32:], -0.5, 0.5) + 1.0)
    torch.testing.assert_close(kernels.glu(gb, kernels.glu_shape("swish", 1.702, 0.5, 0.5, 1.0)).float().cpu(), w2, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(kernels.glu(gu, "silu").cpu(), g * plain.sigmoid(g) * u, rtol=1e-5, atol=1e-6)
    # the unit in the epilogue of the two products that have one: a few rows, and a prompt's rows; into columns of a
    # wider matrix
    from garlic_inference_b200.ops import glu_product, linear
    w = (torch.randn(2 * 96, 64, device="cuda") * 0.3).bfloat16()
    unit = kernels.glu_shape("swish", 1.702, 0.9, 0.9, 1.0)
    for rows in (3, 8, 700):
        x = torch.randn(rows, 64, device="cuda").bfloat16()
        want = kernels.glu(linear(x, w), unit).float().cpu()
        wide = torch.zeros(rows, 96 + 32, device="cuda", dtype=torch.bfloat16)
        got = glu_product(x, w, unit, out=wide[:, 32:])
        torch.testing.assert_close(got.float().cpu(), want, rtol=2e-2, atol=2e-2)
        assert float(wide[:, :32].abs().max()) == 0.0
        torch.testing.assert_close(glu_product(x, w, unit).float().cpu(), want, rtol=2e-2, atol=2e-2)
    kernels.check_bounded_waits(torch.device("cuda", 0))


def test_router_over_all_experts_with_groups_and_the_gated_experts():
    from garlic_inference_b200.ops import kernels
    torch.manual_seed(2)
    for n, E, top, groups, keep, scale in ((45, 12, 5, 4, 2, 2.5), (7, 6, 3, 3, 2, 1.0), (300, 64, 6, 8, 3, 0.5),
                                           (5, 1, 1, 1, 1, 1.0), (9, 40, 40, 5, 5, 1.0), (11, 8, 2, 8, 4, 3.0)):
        z = torch.randn(n, E, device="cuda") * 2
        router = {"experts": E, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}
        idx, wt = kernels.router_select(z, top, groups, keep, scale)
        ri, rw = plain.route(z.cpu(), router)
        assert torch.equal(idx.cpu().long(), ri), f"{E} experts, {groups} groups"
        torch.testing.assert_close(wt.cpu(), rw, rtol=1e-5, atol=1e-7)
    z = torch.log(torch.tensor([[0.25, 0.05, 0.3, 0.02, 0.2, 0.18]])).cuda()
    idx, wt = kernels.router_select(z, 3, 3, 2, 2.0)               # the third best expert sits in a group that leaves
    assert idx.tolist() == [[2, 0, 1]] and torch.allclose(wt.cpu(), torch.tensor([[0.6, 0.5, 0.1]]), atol=1e-6)
    n, E, top, hid, ff = 6, 7, 3, 40, 24
    x = torch.randn(n, hid, device="cuda")
    up, down = torch.randn(E, 2 * ff, hid, device="cuda") * 0.3, torch.randn(E, hid, ff, device="cuda") * 0.3
    idx = torch.stack([torch.randperm(E)[:top] for _ in range(n)]).to(torch.int32).cuda()
    wt = torch.rand(n, top, device="cuda")
    unit = kernels.glu_shape("swish", 1.702, 0.8, 0.8, 1.0)
    want = torch.zeros(n, hid)
    for e in range(E):
        y = plain.swish_glu(x.cpu(), up[e, :ff].cpu(), up[e, ff:].cpu(), down[e].cpu(), 0.8)
        want += y * (wt.cpu() * (idx.cpu() == e)).sum(-1, keepdim=True)
    torch.testing.assert_close(kernels.moe_rowwise(x, up, down, idx, wt, unit).cpu(), want, rtol=1e-4, atol=1e-4)


def test_routed_experts_few_rows_and_many_rows_agree(folder):
    """The part's two ways (row by row for a few tokens, expert by expert for many) on the same rows."""
    from garlic_inference_b200.parts import Runtime, StepContext, part_class
    from garlic_inference_b200.weights import Checkpoint
    ck = Checkpoint(folder("moe"))
    cfg = td.make_config("moe")
    spec = cfg.plan().layers[0].feed_forward

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
    torch.testing.assert_close(many.cpu(), plain.moe_ff(x.cpu(), w, td.config_dict("moe")["layers"][0]["mlp"]), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cache_rows_queries_and_a_key_that_stands_out(dtype):
    """The kernel between projections and attention in the half layout, with queries from a matrix of their own and
    pages out of order; then attention over those rows with one far key made to win: the query's rotated part and
    that key's are made large and parallel after their turns, so the softmax puts nearly everything on that key,
    whether it sits at a page's first or last row, at position 0 or hundreds of keys back; decode kernel, exact-order
    kernel and (bfloat16) the product form."""
    from garlic_inference_b200.ops import kernels
    torch.manual_seed(3)
    H, d, dr, rank, n_rot, base, page, T = 5, 12, 8, 24, 6, 50.0, 16, 300
    row = 40                                   # the latent, the key part and 8 columns of padding
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    q_src = torch.randn(T, H * (d + dr) + 5, device="cuda").to(dtype)[:, 5:]
    kv_src = torch.randn(T, 7 + rank + dr, device="cuda").to(dtype)
    q_lat = torch.randn(T, H, rank, device="cuda").to(dtype)
    norm_w = (1 + 0.1 * torch.randn(rank, device="cuda")).to(dtype)
    freq = torch.tensor([base ** (-2.0 * i / n_rot) for i in range(n_rot // 2)], dtype=torch.float32, device="cuda")
    n_pages = -(-T // page)
    order = torch.randperm(n_pages + 3)[:n_pages]
    table = torch.full((2, n_pages + 1), -1, dtype=torch.int32, device="cuda")
    table[1, :n_pages] = order.to(torch.int32)
    pool = torch.zeros(n_pages + 3, 1, page, row, device="cuda", dtype=dtype)
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    slot = torch.ones(T, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    q_rows = kernels.latent_prepare(q_src, 0, kv_src, 7, q_lat, norm_w, 1e-5, freq, 1.0, n_rot, pos, slot, table, pool, H, d,
                                    dr, rank, status, half_layout=True)
    cached = pool[order.cuda()].reshape(-1, row)[:T].float().cpu()
    c = plain.rms_norm(kv_src[:, 7:7 + rank].float().cpu(), norm_w.float().cpu(), 1e-5)
    kr = plain.turn_halves(kv_src[:, 7 + rank:].float().cpu(), n_rot, base)
    torch.testing.assert_close(cached[:, :rank], c, **tol)
    torch.testing.assert_close(cached[:, rank:rank + dr], kr, **tol)
    assert float(cached[:, rank + dr:].abs().max()) == 0.0
    qr = plain.turn_halves(q_src.float().cpu().view(T, H, d + dr)[:, :, d:], n_rot, base)
    torch.testing.assert_close(q_rows.float().cpu()[:, :, rank:rank + dr], qr, **tol)
    torch.testing.assert_close(q_rows.float().cpu()[:, :, :rank], q_lat.float().cpu(), **tol)
    # a layer on borrowed rows: the same queries, nothing written
    before = pool.clone()
    q2 = kernels.latent_prepare(q_src, 0, None, 0, q_lat, None, 1e-5, freq, 1.0, n_rot, pos, slot, table, pool, H, d, dr,
                                rank, status, append=False, half_layout=True)
    assert torch.equal(q2, q_rows) and torch.equal(pool, before)
    # one key wins: rows written by hand
    rows_all = pool[order.cuda()].reshape(-1, row)
    for far in (0, 15, 16, 31, 130):
        rows = (torch.randn(T, row) * 0.3)
        rows[:, rank + dr:] = 0
        rows[far, rank:rank + dr] = 6.0
        flat = pool.view(-1, row)
        idx = (order[:, None] * page + torch.arange(page)[None, :]).reshape(-1)[:T]
        flat[idx.cuda()] = rows.cuda().to(dtype)
        q = torch.randn(T, H, row) * 0.3
        q[:, :, rank:rank + dr] = 1.0
        q[:, :, rank + dr:] = 0
        q = q.cuda().to(dtype)
        keys = flat[idx.cuda()].float().cpu()
        s = torch.einsum("thr,jr->htj", q.float().cpu(), keys) * 0.7
        want = torch.einsum("htj,jr->thr", plain.causal_softmax(s), keys[:, :rank])
        seen_far = want[max(far, 200):] - keys[far, :rank]
        assert float(seen_far.abs().max()) < 1e-3, "nearly all the weight is on the far key"
        got = kernels.attention_generic(q, pool, pool, table, pos, slot, 0.7, 0, status, value_dim=rank)
        torch.testing.assert_close(got.float().cpu().view(T, H, rank), want, **tol)
        if dtype == torch.bfloat16:
            last = torch.tensor([T - 1, 201, far], device="cuda")
            one = kernels.latent_decode(q[last].contiguous(), pool, table, pos[last].contiguous(), slot[last].contiguous(), 0.7,
                                        None, rank, status, n_splits=3)
            torch.testing.assert_close(one.float().cpu().view(3, H, rank), want[last.cpu()], **tol)
    assert int(status.item()) == 0
