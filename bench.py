#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-8B layer sizes with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

One JSON line on stdout.  `value` is decoded tokens a second at batch 8 with 2,048 cached tokens
per sequence (a step = one decode step of the whole batch), timed on the device with the sampler's
tokens fed back on the device; `e2e` is the same through `LanguageModel.generate` (prompts and
generated ids on the host, every step's ids read back), over the last K of W + K + 1 steps.  The
defaults are 128 steps after 32 warm-up steps: the first twenty or so decode steps right after the prompt
passes take 4.1 to 4.4 ms instead of 3.8 (measured; they do not when the GPU rests half a second in
between, so it is the state the power cap leaves the GPU in, not the engine).  `prefill` is one 2,048-token prompt, `points` decoding at batch 1 and 64, `roofline` the bytes a
decode step has to read (every weight once, the cache of the live requests) over its time against the measured copy bandwidth.

The library runs on one GPU: for --gpus > 1 a line says so and the exit code is 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# layer sizes of the benchmark configuration (Qwen3-8B): 36 layers of hidden 4096, 32 query and 8
# key/value heads of 128, feed-forward 12288, vocabulary 151936, separate head
QWEN3_8B = dict(hidden_size=4096, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, intermediate_size=12288, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                max_position_embeddings=40960, tie_word_embeddings=False)
CONTEXT = 4096          # tokens per sequence the benchmark's context allows
CACHED = 2048           # tokens each sequence holds when decoding is timed
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            p = json.load(open(path))
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                    "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained") or 0) or None, "source": "measured"}
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi in the background while a region is timed (reads only; nothing is set).  Every sample carries
    nvidia-smi's own wall-clock time, so that a summary can be taken over a part of the sampled time."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")

    def __init__(self, gpu_id: str, period_ms: int = 100):
        self.gpu_id, self.period_ms, self.proc, self.lines = gpu_id, period_ms, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.gpu_id, f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        self.lines += [l for l in out.splitlines() if l.strip()]
        self.proc = None

    def summary(self, since: float = None, until: float = None):
        """Median SM clock and the reasons seen, over all samples or over those taken between two time.time() values."""
        import datetime
        sm, mx, watts, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            try:
                if since is not None or until is not None:
                    t = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    if (since is not None and t < since) or (until is not None and t > until):
                        continue
                sm.append(float(f[1])), mx.append(float(f[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, f[3:7]):
                if v.lower() == "active":
                    reasons.add(name)
            try:
                watts.append(float(f[7]))
            except (ValueError, IndexError):
                pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
        if watts:
            out["watts"] = statistics.median(watts)
        return out


def decode_step_bytes(cfg, n_layers, batch, context_tokens):
    """Bytes one decode step has to read: every weight it uses once (bfloat16), the embedding rows of the
    batch, and the keys and values of the live requests."""
    h, d = cfg["hidden_size"], cfg["head_dim"]
    n_q, n_kv, inter, vocab = (cfg[k] for k in ("num_attention_heads", "num_key_value_heads", "intermediate_size",
                                                "vocab_size"))
    per_layer = ((n_q + 2 * n_kv) * d * h + h * n_q * d + 3 * inter * h + 2 * h + 2 * d) * 2
    weights = n_layers * per_layer + (vocab * h + h) * 2 + batch * h * 2
    kv = batch * context_tokens * n_layers * 2 * n_kv * d * 2
    return weights + kv, weights, kv


def prefill_flops(cfg, n_layers, tokens):
    h, d = cfg["hidden_size"], cfg["head_dim"]
    n_q, n_kv, inter, vocab = (cfg[k] for k in ("num_attention_heads", "num_key_value_heads", "intermediate_size",
                                                "vocab_size"))
    linear = 2 * tokens * ((n_q + 2 * n_kv) * d * h + h * n_q * d + 3 * inter * h)
    attn = 4 * n_q * d * tokens * (tokens + 1) // 2
    return n_layers * (linear + attn) + 2 * vocab * h


REFERENCE_RUNNER = os.path.join(ROOT, "baseline", "_ref", "bin", "reference_runner")


def write_reference_model(folder, n_layers):
    """An 8B-size folder for upstream's loader: the same tensors and shapes as the benchmark model, values
    N(0, 0.02) drawn by torch on the GPU, norm weights 1, and `tie_word_embeddings` true because upstream
    always uses the embedding table as the head (src/models/qwen3/qwen3.cpp:58): a decode step reads the same
    bytes.  Nothing of this repository's compiled library is used."""
    import torch
    from garlic_inference_b200 import Qwen3Config
    from garlic_inference_b200.engine.model import wanted_tensors
    from garlic_inference_b200.weights.safetensors_io import write_safetensors_lazy
    cfg = Qwen3Config(**{**QWEN3_8B, "num_hidden_layers": n_layers, "tie_word_embeddings": True})
    wants = wanted_tensors(cfg.plan())
    gen = torch.Generator(device="cuda").manual_seed(0)

    def make(name):
        w = wants[name]
        if w.role == "norm":
            return torch.ones(tuple(w.shape), dtype=torch.bfloat16)
        t = torch.randn(tuple(w.shape), generator=gen, device="cuda", dtype=torch.bfloat16).mul_(0.02)
        return t.cpu()

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    write_safetensors_lazy(os.path.join(folder, "model.safetensors"),
                           {n: (torch.bfloat16, tuple(w.shape)) for n, w in wants.items()}, make)
    torch.cuda.empty_cache()


def reference_arm(args) -> int:
    """Upstream's own dense Qwen3 code (built unmodified for sm_100a by baseline/build_reference.py, with the
    driver baseline/reference_driver.cpp) on the benchmark's workload: the same JSON line, `impl: reference`."""
    import shutil
    import tempfile

    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    if not os.path.isfile(REFERENCE_RUNNER):
        src = os.environ.get("GARLIC_REFERENCE_SRC", os.path.join(os.path.dirname(ROOT), "reference"))
        if not os.path.isdir(src):
            return unavailable("baseline/_ref/bin/reference_runner is not built and there is no upstream checkout "
                               "here to build it from (baseline/build_reference.py)")
        r = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "build_reference.py"), "--src", src],
                           capture_output=True, text=True)
        if r.returncode != 0 or not os.path.isfile(REFERENCE_RUNNER):
            return unavailable("building upstream's dense path failed: " + (r.stderr or r.stdout).strip()[-300:].replace("\n", " "))
    import torch
    if not torch.cuda.is_available():
        return unavailable("no GPU here")
    K, W = args.steps, max(args.warmup, 3)
    n_layers = args.layers or QWEN3_8B["num_hidden_layers"]
    pk = peaks()
    props = torch.cuda.get_device_properties(0)
    gpu_id = "GPU-" + str(props.uuid) if getattr(props, "uuid", None) else "0"
    need = 2.2 * (n_layers * 385.9e6 + 1.25e9)                  # the file, with room to spare
    base = next((d for d in ("/dev/shm", tempfile.gettempdir()) if os.path.isdir(d) and shutil.disk_usage(d).free > need), None)
    if base is None:
        return unavailable("no temporary folder with %.0f GB free for the model file" % (need / 1e9))
    folder = tempfile.mkdtemp(prefix="garlic_ref_model_", dir=base)
    try:
        t0 = time.time()
        write_reference_model(folder, n_layers)
        print(f"bench.py: wrote the model folder in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)

        def run(batch, chunk, steps, warmup, repeats=0, clocks=None):
            cmd = [REFERENCE_RUNNER, folder, "--batch", str(batch), "--prompt-len", str(CACHED), "--chunk", str(chunk),
                   "--steps", str(steps), "--warmup", str(warmup), "--prefill-repeats", str(repeats)]
            if clocks:
                clocks.start()
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=1200)
            if clocks:
                clocks.stop()
            if r.returncode != 0:
                raise RuntimeError(f"reference_runner exited with {r.returncode}: {(r.stderr or r.stdout).strip()[-300:]}")
            return json.loads(r.stdout.strip().splitlines()[-1])

        clocks = ClockSampler(gpu_id)
        try:
            main_run = run(args.batch, 1024 if args.batch * CACHED * QWEN3_8B["vocab_size"] >= 2 ** 31 else CACHED, K, W,
                           clocks=clocks)
            pre = run(1, PREFILL_TOKENS, 0, 0, repeats=4)
            points = {}
            for b, chunk in (() if args.no_points else ((1, CACHED), (64, 128))):
                try:                                   # a point that cannot run (memory) leaves the others standing
                    points[f"decode_b{b}"] = b * 1e3 / run(b, chunk, K, W)["decode_ms_per_step"]
                except RuntimeError as e:
                    points[f"decode_b{b}_unavailable"] = str(e)[:200]
        except (RuntimeError, subprocess.TimeoutExpired, ValueError, IndexError) as e:
            return unavailable(str(e).replace("\n", " ")[:400])
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    ms = main_run["decode_ms_per_step"]
    pre_ms = statistics.median(pre["prefill_ms"][1:])
    total_b, weight_b, _ = decode_step_bytes(QWEN3_8B, n_layers, args.batch, CACHED + W + (K + 1) / 2)
    achieved = total_b / (ms / 1e3) / 1e9
    line = {
        "impl": "reference",
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-8B layer sizes, {CACHED} cached tokens per sequence)",
        "value": args.batch * 1e3 / ms, "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02) in a model folder, token ids from a counter; the head is tied "
                "because upstream always ties it (the same bytes are read per step)",
        "config": {"model": "Qwen3-8B layer sizes", "global_batch": args.batch, "seq_len": CONTEXT,
                   "cached_tokens": CACHED, "parallelism": "none (1 GPU)", "layers_run": n_layers,
                   "layers_config": QWEN3_8B["num_hidden_layers"], "hidden_size": 4096, "n_heads": 32,
                   "n_kv_heads": 8, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936,
                   "page_size": 32, "sampling": "upstream's argmax, result read by the host every step",
                   "prompt_chunk": main_run["chunk"],
                   "l2": "inputs exceed L2: a step reads %.1f GB of weights" % (weight_b / 1e9)},
        "clocks": clocks.summary(),
        # upstream's loop is synchronous: every step copies positions and block tables to the device and reads the
        # argmax back, so the wall clock over the same steps is its end-to-end figure
        "e2e": {"value": args.batch * 1e3 / main_run["decode_wall_ms_per_step"], "unit": "tokens/s",
                "h2d_bytes_per_step": main_run["h2d_bytes_per_step"], "d2h_bytes_per_step": main_run["d2h_bytes_per_step"]},
        "gpu_launches": 0,
        "prefill": {"value": PREFILL_TOKENS / (pre_ms / 1e3), "tokens": PREFILL_TOKENS, "ms": pre_ms,
                    "frac": (prefill_flops(QWEN3_8B, n_layers, PREFILL_TOKENS) + 2 * (PREFILL_TOKENS - 1) * 151936 * 4096)
                    / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12),
                    "note": "upstream computes logits at all 2,048 positions and reads 2,048 argmax results back"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": total_b, "peaks": pk["source"]},
        "points": points,
        "memory": {"free_gb_after_prompt": main_run["free_gb_after_prompt"], "free_gb_at_end": main_run["free_gb_at_end"]},
    }
    print(json.dumps(line))
    return 0


# the two larger workloads (layer sizes of Qwen3-14B and Qwen3-32B), run through `generate()`
LARGER = {
    "qwen3_14b": dict(cfg=dict(hidden_size=5120, num_hidden_layers=40, num_attention_heads=40, num_key_value_heads=8,
                               head_dim=128, intermediate_size=17408, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                               max_position_embeddings=40960, tie_word_embeddings=False),
                      batch=16, prompt=(256, 2048), new_tokens=512),
    "qwen3_32b": dict(cfg=dict(hidden_size=5120, num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8,
                               head_dim=128, intermediate_size=25600, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                               max_position_embeddings=40960, tie_word_embeddings=False),
                      batch=32, prompt=(1024, 1024), new_tokens=1024),
}


def larger_workloads(first_model, pk, gpu_id) -> dict:
    """Batch 16 with prompts uniform in [256, 2,048] then 512 decode steps at Qwen3-14B layer sizes; batch 32 with
    prompts of 1,024 then 1,024 decode steps at Qwen3-32B layer sizes (65.5 GB of weights).  Random weights, all
    layers, through `LanguageModel.generate` (host ids in and out).  Decode figures are over all decode steps."""
    import gc
    import torch
    from garlic_inference_b200 import LanguageModel, Qwen3Config
    # the benchmark model leaves the device before the larger ones arrive
    first_model.engine.graphs = None
    first_model.engine.cache = None
    first_model.engine.model = None
    first_model.model = None
    gc.collect()
    torch.cuda.empty_cache()
    out = {}
    gen = torch.Generator().manual_seed(1)
    for name, w in LARGER.items():
        cfg = Qwen3Config(**w["cfg"])
        lo, hi = w["prompt"]
        lens = [lo] * w["batch"] if lo == hi else torch.randint(lo, hi + 1, (w["batch"],), generator=gen).tolist()
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for n in lens]
        per_seq = [-(-(n + w["new_tokens"]) // 64) * 64 for n in lens]
        try:
            model = LanguageModel.from_random(cfg, seed=0, device=0, dtype="bfloat16", max_tokens=sum(per_seq) + 64)
            model.generate([p[:64] for p in prompts], max_new_tokens=8)             # records the decode step, warms the path
            clocks = ClockSampler(gpu_id, period_ms=50)
            clocks.start()
            toks = model.generate(prompts, max_new_tokens=w["new_tokens"])
            clocks.stop()
            st = model.last_stats
            assert all(len(t) == w["new_tokens"] for t in toks)
            steps = len(st.step_times) - 1                                          # decode steps (the first time is the prompt step's)
            seconds = st.step_times[-1] - st.step_times[0]
            ctx = sum(lens) / len(lens) + steps / 2
            total_b, weight_b, kv_b = decode_step_bytes(w["cfg"], cfg.num_hidden_layers, w["batch"], ctx)
            ms = 1e3 * seconds / steps
            out[name] = {"batch": w["batch"], "prompt_tokens": sum(lens), "decode_steps": steps, "layers": cfg.num_hidden_layers,
                         "decode_tok_s": w["batch"] * steps / seconds, "ms_per_step": ms,
                         "prefill_tok_s": sum(lens) / st.prefill_seconds if st.prefill_seconds else None,
                         "bytes_per_step": total_b, "hbm_frac": total_b / (ms / 1e3) / 1e9 / pk["hbm_gbs"],
                         "weights_gb": weight_b / 1e9, "sm_mhz": clocks.summary().get("sm_mhz")}
            model.engine.check()
        except Exception as e:                                                      # a point that cannot run leaves the line standing
            out[name] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        model = None
        gc.collect()
        torch.cuda.empty_cache()
    return out


def study_prefill_clocks(model, prompt, gpu_id, flops) -> int:
    """How a prompt step's time follows the clock: the first steps of a burst run at the full clock, then the power
    cap pulls the clock down and the step time goes up with it."""
    import datetime
    import torch
    eng = model.engine
    clocks = ClockSampler(gpu_id, period_ms=20)
    slots = [eng.alloc_slot() for _ in range(2)]
    model.step([(slots[0], prompt, [len(prompt) - 1])])                     # warm the path
    eng.free_slot(slots[0])
    torch.cuda.synchronize()
    time.sleep(1.0)                                                         # let the GPU rest: the burst starts cool
    clocks.start()
    time.sleep(0.1)
    rows, events = [], []
    t_wall0 = time.time()
    for i in range(40):
        s = eng.alloc_slot()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        model.step([(s, prompt, [len(prompt) - 1])])
        b.record()
        eng.free_slot(s)
        events.append((a, b))
    torch.cuda.synchronize()
    t_wall1 = time.time()
    clocks.stop()
    samples = []
    for l in clocks.lines:
        f = [x.strip() for x in l.split(",")]
        try:
            samples.append((datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp(), float(f[1]), float(f[7])))
        except (ValueError, IndexError):
            pass
    ms = [a.elapsed_time(b) for a, b in events]
    t = t_wall0
    print("step   ms     TFLOP/s   sm MHz   W      ms x GHz")
    for i, m in enumerate(ms):
        mid = t + m / 2e3
        near = min(samples, key=lambda s: abs(s[0] - mid)) if samples else (0, float("nan"), float("nan"))
        print(f"{i:3d}  {m:6.2f}  {flops / m / 1e9:8.0f}  {near[1]:7.0f}  {near[2]:5.0f}  {m * near[1] / 1e3:7.2f}")
        t += (t_wall1 - t_wall0) / len(ms)
    return 0


# ---- the Fivitar design beside Qwen3 at equal layer sizes ------------------------------------------
def fivitar_config_dict(width, heads, ff, vocab, n_layers, head_dim=128, kv_rank=512, rot_dim=64):
    """`n_layers` layers that cycle through the three mixers, every one with a feed-forward, at sizes of a real
    model's layers: heads of `head_dim` keys and values, a latent of `kv_rank` with a rotated part of `rot_dim`."""
    def layer(i):
        kind = ("delta", "lightning", "latent_attention")[i % 3]
        if kind == "delta":
            mixer = {"heads": heads, "kv_heads": max(1, heads // 2), "dim": head_dim, "vdim": head_dim, "conv": 4}
        elif kind == "lightning":
            mixer = {"heads": heads, "dim": head_dim, "vdim": head_dim,
                     "decay": [1.0 - 2.0 ** (-5 - 3 * h / max(1, heads - 1)) for h in range(heads)]}
        else:
            mixer = {"heads": heads, "dim": head_dim, "rot_dim": rot_dim, "vdim": head_dim, "kv_rank": kv_rank,
                     "scale": (head_dim + rot_dim) ** -0.5,
                     "rot": {"base": 10000.0, "dims": rot_dim,
                             "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
        return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff}}
    return {"architecture": "Fivitar", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "layers": [layer(i) for i in range(n_layers)]}


def study_fivitar(args, pk) -> int:
    """Prefill (one prompt of 2,048 tokens) and decode (batches of 1, 8 and 64 with 2,048 cached tokens each)
    of Fivitar models with random weights, beside Qwen3 models of the same width, depth, heads and feed-forward
    parameters, and every kernel of both timed alone at those sizes.  One JSON line."""
    import torch
    from garlic_inference_b200 import LanguageModel, Qwen3Config
    from garlic_inference_b200.config import FivitarConfig
    from garlic_inference_b200.ops import counters, kernels
    from garlic_inference_b200.sampling import SamplingParams
    K, W = min(args.steps, 64), max(min(args.warmup, 8), 3)
    torch.cuda.set_device(0)
    greedy = SamplingParams()
    gen = torch.Generator().manual_seed(0)
    sizes = [("1b", 2048, 16, 8192, 32000, 6), ("8b", 4096, 32, 18432, 32000, 6)]
    out = {"study": "fivitar", "dtype": "bfloat16", "data": "synthetic", "steps": K, "warmup": W,
           "peaks": pk, "models": {}, "kernels": {}}

    def timed(fn, reps=5, warm=3):
        for _ in range(warm):
            fn()
        flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda")
        ms = []
        for _ in range(reps):
            flush.zero_()                                  # larger than L2: the next run starts cold
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            ms.append(a.elapsed_time(b))
        return statistics.median(ms)

    def run_model(cfg, vocab):
        per_seq = -(-(CACHED + W + K + 8) // 64) * 64
        model = LanguageModel.from_random(cfg, seed=0, device=0, dtype="bfloat16", max_tokens=64 * per_seq,
                                          max_slots=64)
        eng, sampler = model.engine, model.sampler
        prompt = lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist()
        res = {"weight_bytes": model.model.weight_bytes()}

        def prefill_once():
            s = eng.alloc_slot()
            model.step([(s, prompt(PREFILL_TOKENS), [PREFILL_TOKENS - 1])])
            eng.free_slot(s)
        ms = timed(prefill_once, reps=5, warm=3)
        res["prefill"] = {"tokens": PREFILL_TOKENS, "ms": round(ms, 3), "tokens_per_s": round(PREFILL_TOKENS / ms * 1e3)}
        for batch in (1, 8, 64):
            slots, firsts = [], []
            for _ in range(batch):
                s = eng.alloc_slot()
                firsts.append(sampler.sample(model.step([(s, prompt(CACHED), [CACHED - 1])]), greedy, [0], [0]))
                slots.append(s)
            toks = torch.cat(firsts)
            for _ in range(W):
                toks = sampler.sample(eng.step_decode_device(slots, toks), greedy, slots, slots)
            torch.cuda.synchronize()
            n0 = counters.launches
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(K):
                toks = sampler.sample(eng.step_decode_device(slots, toks), greedy, slots, slots)
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / K
            state = eng.cache.state_bytes_per_slot * batch + eng.cache.bytes_per_token() * batch * CACHED
            res[f"decode_b{batch}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(batch / ms * 1e3),
                                       "launches_per_step": (counters.launches - n0) // K,
                                       "bytes_read": res["weight_bytes"] + state,
                                       "of_measured_copy": round((res["weight_bytes"] + state) / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 3)}
            for s in slots:
                eng.free_slot(s)
        eng.check()
        del model
        torch.cuda.empty_cache()
        return res

    for label, width, heads, ff, vocab, n_layers in sizes:
        fcfg = FivitarConfig.from_dict(fivitar_config_dict(width, heads, ff, vocab, n_layers))
        inter = -(-(2 * ff // 3) // 256) * 256                      # three matrices instead of two: equal parameters
        qcfg = Qwen3Config(hidden_size=width, num_hidden_layers=n_layers, num_attention_heads=heads,
                           num_key_value_heads=max(1, heads // 4), head_dim=128, intermediate_size=inter,
                           vocab_size=vocab, max_position_embeddings=CONTEXT * 2)
        out["models"][label] = {"width": width, "heads": heads, "ff": ff, "layers": n_layers,
                                "fivitar": run_model(fcfg, vocab), "qwen3": run_model(qcfg, vocab)}

    # ---- the mixers' kernels alone, at the larger size: one prompt of 2,048 tokens, and 8 single tokens ----
    H, d, dv, rank, dr, T, page = 32, 128, 128, 512, 64, PREFILL_TOKENS, 64
    dev = "cuda"
    bf = lambda *shape: torch.randn(*shape, device=dev, dtype=torch.bfloat16) * 0.5
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    from garlic_inference_b200.parts.linear_attention import scan_state_floats
    sf = H * scan_state_floats(d, dv)
    C = 2 * (H // 2) * d + H * dv
    kern = out["kernels"]

    def note(name, ms, flops=0.0, bytes_=0.0):
        kern[name] = {"ms": round(ms, 4)}
        if flops:
            kern[name]["tflops"] = round(flops / ms / 1e9, 2)
        if bytes_:
            kern[name]["gbs"] = round(bytes_ / ms / 1e6, 1)
            kern[name]["of_measured_copy"] = round(bytes_ / ms / 1e6 / pk["hbm_gbs"], 3)

    for n_rows, tag, spans, slots in ((T, "prefill2048", i32([[0, 0, T]]), i32([0] * T)),
                                      (8, "decode_b8", None, i32(list(range(8))))):
        state = torch.zeros(9, sf + 3 * C + 8, device=dev)
        qkvg = bf(n_rows, 4 * H * d)
        decay = torch.full((H,), 0.99, device=dev)
        ms = timed(lambda: kernels.decay_scan(qkvg, (0, H * d, 2 * H * d), decay, state[:, :sf], spans, slots, H, d, dv))
        seqs = 1 if spans is not None else 8
        note(f"decay_scan_{tag}", ms, flops=4.0 * n_rows * H * d * dv,
             bytes_=seqs * 2 * sf * 4 + n_rows * (3 * H * d * 2 + H * dv * 4))
        conv_out = torch.randn(n_rows, C, device=dev)
        ba = torch.randn(n_rows, 2 * H, device=dev)
        A, dtb = torch.zeros(H, device=dev), torch.zeros(H, device=dev)
        ms = timed(lambda: kernels.delta_scan(conv_out, (0, H // 2 * d, H * d), ba, (0, H), A, dtb, state[:, :sf], spans,
                                              slots, H, H // 2, d, dv, 1e-6))
        note(f"delta_scan_{tag}", ms, flops=8.0 * n_rows * H * d * dv,
             bytes_=seqs * 2 * sf * 4 + n_rows * (C * 4 + H * dv * 4))
        x = bf(n_rows, C)
        taps = bf(C, 4)
        ms = timed(lambda: (kernels.causal_conv_silu(x, taps, state[:, sf:], slots),
                            kernels.conv_state_update(x, 4, state[:, sf:], slots)))
        note(f"conv_silu_and_state_{tag}", ms, bytes_=n_rows * C * (2 + 4))
    # attention: the latent rows of one sequence of 2,048 (prefill) and of 8 sequences of 2,048 (decode)
    row = rank + dr
    pool = bf(8 * T // page, 1, page, row)
    table = torch.arange(8 * T // page, dtype=torch.int32, device=dev).view(8, T // page)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    sinks = torch.zeros(H, device=dev)
    q = bf(T, H, row)
    pos, slot0 = torch.arange(T, dtype=torch.int32, device=dev), i32([0] * T)
    ms = timed(lambda: kernels.attention_generic(q, pool, pool, table, pos, slot0, 0.07, 0, status, sinks=sinks,
                                                 value_dim=rank), reps=3, warm=1)
    note("latent_attention_prefill2048_exact_order", ms, flops=2.0 * H * (row + rank) * T * (T + 1) / 2)
    rows = pool.view(-1, page, row)[:T // page].reshape(T, row)

    def by_products():                       # what the mixer runs for a prompt in bfloat16: blocks of 1,024 tokens
        for q0 in range(0, T, 1024):
            scores = torch.mm(q[q0:q0 + 1024].view(1024 * H, row), rows[:q0 + 1024].t(), out_dtype=torch.float32)
            w = kernels.causal_sink_softmax(scores, H, q0, 0.07, sinks, torch.bfloat16)
            torch.mm(w, rows[:q0 + 1024, :rank])
    ms = timed(by_products)
    note("latent_attention_prefill2048_products", ms, flops=2.0 * H * (row + rank) * T * (T + 1) / 2)
    q8, pos8, slots8 = bf(8, H, row), i32([T - 1] * 8), i32(list(range(8)))
    ms = timed(lambda: kernels.attention_generic(q8, pool, pool, table, pos8, slots8, 0.07, 0, status,
                                                 sinks=sinks, value_dim=rank))
    note("latent_attention_decode_b8_exact_order", ms, bytes_=8 * T * row * 2)
    ms = timed(lambda: kernels.latent_decode(q8, pool, table, pos8, slots8, 0.07, sinks, rank, status))
    note("latent_attention_decode_b8_shared_rows", ms, flops=2.0 * 8 * H * (row + rank) * T, bytes_=8 * T * row * 2)
    # the closest existing kernels: grouped-query flash attention over 2,048 tokens, and split-KV decoding
    from garlic_inference_b200.parts.attention import query_runs
    from garlic_inference_b200.parts import StepShape
    n_kv = 8
    kp, vp = bf(8 * T // page, n_kv, page, 128), bf(8 * T // page, n_kv, page, 128)
    qq = bf(T, H, 128)
    runs = torch.from_numpy(query_runs(StepShape([0], [0], [T], [0], False), 128)).to(dev)
    ms = timed(lambda: kernels.attention_prefill_tcgen05(qq, kp, vp, table, runs, 0.088, 0, rows_covered=True))
    note("gqa_attention_prefill2048_tcgen05", ms, flops=4.0 * H * 128 * T * (T + 1) / 2)
    qd = bf(8, H, 128)
    ms = timed(lambda: kernels.attention_decode_tcgen05(qd, kp, vp, table, pos8, slots8, 0.088, 0))
    note("gqa_attention_decode_b8_tcgen05", ms, bytes_=8 * T * 2 * n_kv * 128 * 2)
    kernels.check_bounded_waits(torch.device("cuda", 0))
    print(json.dumps(out))
    return 0


# ---- the Zogulorn design beside Qwen3 at equal layer sizes -----------------------------------------
def zogulorn_config_dict(width, heads, ff, vocab, n_layers, head_dim=128, chunk=1024, experts=16, top=2):
    """`n_layers` layers that cycle through parallel + dense, attention + experts, parallel + experts and an
    attention on the first attention's keys and values + dense, at sizes of a real model's layers."""
    kv = max(1, heads // 4)
    left = {"heads": heads, "kv_heads": kv, "dim": head_dim, "vdim": head_dim, "mask": {"size": chunk},
            "rot": {"base": 250000.0, "dims": head_dim}, "scale": head_dim ** -0.5}
    right = {"heads": heads // 2, "kv_heads": max(1, heads // 4), "dim": head_dim, "vdim": head_dim, "conv": 4,
             "rank": max(8, width // 16)}
    par = {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 0.6, "right_scale": 1.1}}
    att = lambda src: {"type": "attention",
                       "mixer": dict({"heads": heads // 2, "kv_heads": max(1, kv // 2), "dim": head_dim // 2,
                                      "vdim": head_dim, "mask": {"size": 2 * chunk}, "conv": 4, "diff": 0.6,
                                      "scale": (head_dim // 2) ** -0.5}, **({"kv_from": src} if src is not None else {}))}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": max(64, ff * 3 // (2 * top) // 64 * 64)}, "router": {"experts": experts, "top": top}}
    layers, first_att = [], None
    for i in range(n_layers):
        k = i % 4
        if k in (0, 2):
            layers.append(dict(par, mlp=dense if k == 0 else moe))
        elif k == 1 or first_att is None:
            first_att = i if first_att is None else first_att
            layers.append(dict(att(None), mlp=moe))
        else:
            layers.append(dict(att(first_att), mlp=dense))
    return {"architecture": "Zogulorn", "vocab": vocab, "width": width, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "layers": layers}


def study_zogulorn(args, pk) -> int:
    """Prefill (one prompt of 2,048 tokens) and decode (batches of 1, 8 and 64 with 2,048 cached tokens each) of
    Zogulorn models with random weights, beside Qwen3 models of the same width, depth and heads with a
    feed-forward of equal active parameters, and the design's kernels timed alone beside the closest kernels of
    the other models.  One JSON line."""
    import torch
    from garlic_inference_b200 import LanguageModel, Qwen3Config
    from garlic_inference_b200.config import ZogulornConfig
    from garlic_inference_b200.ops import counters, kernels
    from garlic_inference_b200.sampling import SamplingParams
    K, W = min(args.steps, 64), max(min(args.warmup, 8), 3)
    torch.cuda.set_device(0)
    greedy = SamplingParams()
    gen = torch.Generator().manual_seed(0)
    sizes = [("1b", 2048, 16, 8192, 32000, 8), ("8b", 4096, 32, 18432, 32000, 4)]
    out = {"study": "zogulorn", "dtype": "bfloat16", "data": "synthetic", "steps": K, "warmup": W,
           "peaks": pk, "models": {}, "kernels": {}}

    def timed(fn, reps=5, warm=3):
        for _ in range(warm):
            fn()
        flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda")
        ms = []
        for _ in range(reps):
            flush.zero_()                                  # larger than L2: the next run starts cold
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            ms.append(a.elapsed_time(b))
        return statistics.median(ms)

    def run_model(cfg, vocab, active_bytes=None):
        per_seq = -(-(CACHED + W + K + 8) // 64) * 64
        model = LanguageModel.from_random(cfg, seed=0, device=0, dtype="bfloat16", max_tokens=64 * per_seq,
                                          max_slots=64)
        eng, sampler = model.engine, model.sampler
        prompt = lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist()
        res = {"weight_bytes": model.model.weight_bytes()}

        def prefill_once():
            s = eng.alloc_slot()
            model.step([(s, prompt(PREFILL_TOKENS), [PREFILL_TOKENS - 1])])
            eng.free_slot(s)
        ms = timed(prefill_once, reps=5, warm=3)
        res["prefill"] = {"tokens": PREFILL_TOKENS, "ms": round(ms, 3), "tokens_per_s": round(PREFILL_TOKENS / ms * 1e3)}
        for batch in (1, 8, 64):
            slots, firsts = [], []
            for _ in range(batch):
                s = eng.alloc_slot()
                firsts.append(sampler.sample(model.step([(s, prompt(CACHED), [CACHED - 1])]), greedy, [0], [0]))
                slots.append(s)
            toks = torch.cat(firsts)
            for _ in range(W):
                toks = sampler.sample(eng.step_decode_device(slots, toks), greedy, slots, slots)
            torch.cuda.synchronize()
            n0 = counters.launches
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(K):
                toks = sampler.sample(eng.step_decode_device(slots, toks), greedy, slots, slots)
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / K
            res[f"decode_b{batch}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(batch / ms * 1e3),
                                       "launches_per_step": (counters.launches - n0) // K}
            for s in slots:
                eng.free_slot(s)
        eng.check()
        del model
        torch.cuda.empty_cache()
        return res

    for label, width, heads, ff, vocab, n_layers in sizes:
        zcfg = ZogulornConfig.from_dict(zogulorn_config_dict(width, heads, ff, vocab, n_layers))
        qcfg = Qwen3Config(hidden_size=width, num_hidden_layers=n_layers, num_attention_heads=heads,
                           num_key_value_heads=max(1, heads // 4), head_dim=128, intermediate_size=ff,
                           vocab_size=vocab, max_position_embeddings=CONTEXT * 2)
        out["models"][label] = {"width": width, "heads": heads, "ff": ff, "layers": n_layers,
                                "zogulorn": run_model(zcfg, vocab), "qwen3": run_model(qcfg, vocab)}

    # ---- the kernels alone, at the larger size: one prompt of 2,048 tokens, and 8 single tokens ----
    width, H, G, d, T, page, chunk = 4096, 32, 8, 128, PREFILL_TOKENS, 64, 1024
    dev = "cuda"
    bf = lambda *shape: torch.randn(*shape, device=dev, dtype=torch.bfloat16) * 0.5
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    from garlic_inference_b200.parts import StepShape
    from garlic_inference_b200.parts.attention import query_runs
    from garlic_inference_b200.parts.linear_attention import scan_state_floats
    kern = out["kernels"]

    def note(name, ms, flops=0.0, bytes_=0.0):
        kern[name] = {"ms": round(ms, 4)}
        if flops:
            kern[name]["tflops"] = round(flops / ms / 1e9, 2)
            kern[name]["of_measured_bf16"] = round(flops / ms / 1e9 / pk["bf16_tflops"], 4)
        if bytes_:
            kern[name]["gbs"] = round(bytes_ / ms / 1e6, 1)
            kern[name]["of_measured_copy"] = round(bytes_ / ms / 1e6 / pk["hbm_gbs"], 3)

    status = torch.zeros(1, dtype=torch.int32, device=dev)
    table = torch.arange(8 * T // page, dtype=torch.int32, device=dev).view(8, T // page)
    pos, slot0 = torch.arange(T, dtype=torch.int32, device=dev), i32([0] * T)
    pos8, slots8 = i32([T - 1] * 8), i32(list(range(8)))
    runs64 = torch.from_numpy(query_runs(StepShape([0], [0], [T], [0], False), 64)).to(dev)
    runs128 = torch.from_numpy(query_runs(StepShape([0], [0], [T], [0], False), 128)).to(dev)
    kp, vp = bf(8 * T // page, G, page, d), bf(8 * T // page, G, page, d)
    q = bf(T, H, d)
    seen = sum(min(p % chunk, p) + 1 for p in range(T))            # (query, key) pairs inside the chunks
    # chunked attention for a prompt: the design's kernel, and the closest kernels (causal over all keys)
    ms = timed(lambda: kernels.attention_prefill_masked_bf16(q, kp, vp, table, runs64, 0.088, chunk=chunk, rows_covered=True))
    note("chunk_attention_prefill2048_mma", ms, flops=4.0 * H * d * seen)
    ms = timed(lambda: kernels.attention_prefill_tcgen05(q, kp, vp, table, runs128, 0.088, 0, rows_covered=True, chunk=chunk))
    note("chunk_attention_prefill2048_tcgen05", ms, flops=4.0 * H * d * seen)
    ms = timed(lambda: kernels.attention_prefill_bf16(q, kp, vp, table, runs64, 0.088, 0, rows_covered=True))
    note("gqa_attention_prefill2048_mma", ms, flops=4.0 * H * d * T * (T + 1) / 2)
    ms = timed(lambda: kernels.attention_prefill_tcgen05(q, kp, vp, table, runs128, 0.088, 0, rows_covered=True))
    note("gqa_attention_prefill2048_tcgen05", ms, flops=4.0 * H * d * T * (T + 1) / 2)
    # differential attention for a prompt: two maps of 64 over values of 128 (exact-order kernel), 16 heads
    Hd, Gd, dd = 16, 4, 64
    kpd, qd2 = bf(8 * T // page, Gd * 2, page, dd), bf(T, Hd * 2, dd)
    vpd = bf(8 * T // page, Gd, page, d)
    seen2 = sum(min(p % (2 * chunk), p) + 1 for p in range(T))
    ms = timed(lambda: kernels.attention_prefill_masked_bf16(qd2, kpd, vpd, table, runs64, 0.125, chunk=2 * chunk, maps=2,
                                                             rows_covered=True))
    note("differential_attention_prefill2048_mma", ms, flops=2.0 * Hd * 2 * (dd + d) * seen2)
    ms = timed(lambda: kernels.attention_masked(qd2, kpd, vpd, table, pos, slot0, 0.125, status, chunk=2 * chunk, maps=2,
                                                out_float32=True), reps=3, warm=1)
    note("differential_attention_prefill2048_exact_order", ms, flops=2.0 * Hd * 2 * (dd + d) * seen2)
    # decode steps: 8 sequences of 2,048 cached tokens
    q8 = bf(8, H, d)
    ms = timed(lambda: kernels.attention_decode_masked_bf16(q8, kp, vp, table, pos8, slots8, 0.088, chunk=chunk))
    note("chunk_attention_decode_b8_mma", ms, bytes_=8 * (T - chunk) * 2 * G * d * 2)
    ms = timed(lambda: kernels.attention_decode_bf16(q8, kp, vp, table, pos8, slots8, 0.088, 0))
    note("gqa_attention_decode_b8_mma", ms, bytes_=8 * T * 2 * G * d * 2)
    ms = timed(lambda: kernels.attention_masked(q8, kp, vp, table, pos8, slots8, 0.088, status, chunk=chunk, out_float32=True))
    note("chunk_attention_decode_b8_exact_order", ms, bytes_=8 * (T - chunk) * 2 * G * d * 2)
    ms = timed(lambda: kernels.attention_decode_tcgen05(q8, kp, vp, table, pos8, slots8, 0.088, 0))
    note("gqa_attention_decode_b8_tcgen05", ms, bytes_=8 * T * 2 * G * d * 2)
    q8d = bf(8, Hd * 2, dd)
    ms = timed(lambda: kernels.attention_decode_masked_bf16(q8d, kpd, vpd, table, pos8, slots8, 0.125, chunk=2 * chunk, maps=2))
    note("differential_attention_decode_b8_mma", ms, bytes_=8 * T * (2 * Gd * dd + Gd * d) * 2)
    # the delta rule's scan with a decay per key channel, beside the one with a decay per head
    Hr, Hk = 16, 8
    sf = Hr * scan_state_floats(d, d)
    C = 2 * Hk * d + Hr * d
    for n_rows, tag, spans, slots in ((T, "prefill2048", i32([[0, 0, T]]), i32([0] * T)),
                                      (8, "decode_b8", None, i32(list(range(8))))):
        state = torch.zeros(9, sf, device=dev)
        conv_out = torch.randn(n_rows, C, device=dev)
        b_log, a_head, a_chan = (torch.randn(n_rows, c, device=dev) for c in (Hr, Hr, Hr * d))
        A, dt_h, dt_c = torch.zeros(Hr, device=dev), torch.zeros(Hr, device=dev), torch.zeros(Hr * d, device=dev)
        seqs = 1 if spans is not None else 8
        bytes_ = seqs * 2 * sf * 4 + n_rows * (C * 4 + Hr * d * 4)
        ms = timed(lambda: kernels.delta_scan(conv_out, (0, Hk * d, 2 * Hk * d), b_log, (0, 0), A, dt_c, state, spans, slots,
                                              Hr, Hk, d, d, 1e-6, channel_decay=True, decay_logits=a_chan))
        note(f"delta_scan_channel_decay_{tag}", ms, flops=8.0 * n_rows * Hr * d * d, bytes_=bytes_ + n_rows * Hr * d * 4)
        ms = timed(lambda: kernels.delta_scan(conv_out, (0, Hk * d, 2 * Hk * d), b_log, (0, 0), A, dt_h, state, spans, slots,
                                              Hr, Hk, d, d, 1e-6, decay_logits=a_head))
        note(f"delta_scan_head_decay_{tag}", ms, flops=8.0 * n_rows * Hr * d * d, bytes_=bytes_)
    # the norm beside RMSNorm, the gated unit beside SwiGLU, at 2,048 rows
    res, delta = torch.randn(T, width, device=dev), bf(T, width)
    w, b, al, ls = bf(width), bf(width), bf(1), bf(width)
    ms = timed(lambda: kernels.add_dyt(delta, ls, res, w, b, al, torch.bfloat16))
    note("scaled_add_dyt_2048", ms, bytes_=T * width * (2 + 4 + 4 + 2))
    ms = timed(lambda: kernels.add_rmsnorm(delta, res, w, 1e-6, torch.bfloat16))
    note("add_rmsnorm_2048", ms, bytes_=T * width * (2 + 4 + 4 + 2))
    gu = bf(T, 2 * 18432)
    ms = timed(lambda: kernels.glu(gu, "gelu_tanh"))
    note("gelu_glu_2048", ms, bytes_=T * 18432 * 6)
    ms = timed(lambda: kernels.swiglu(gu))
    note("swiglu_2048", ms, bytes_=T * 18432 * 6)
    # routed experts: 16 experts of 13,824, 2 chosen; 8 rows (row by row) and 2,048 rows (expert by expert), beside a
    # dense gated feed-forward of the same active size run through the same products
    from garlic_inference_b200.ops import linear
    from garlic_inference_b200.parts import Runtime, StepContext, part_class
    E, top, eff = 16, 2, 13824

    class Load:
        def dtype(self, *a):
            return torch.bfloat16

        def __call__(self, n, out=None):
            shape = (E, width) if n == "router" else ((eff, width) if n.endswith("up") else (width, eff))
            t = bf(*shape) * 0.05
            return t if out is None else out.copy_(t)

    part = part_class("routed_experts")(dict(hidden_size=width, expert_size=eff, n_experts=E, top=top), Load(),
                                        Runtime(torch.bfloat16, torch.device(dev)))
    z = i32([0])
    for n_rows in (1, 8, 64, T):
        x = bf(n_rows, width)
        ctx = StepContext(n_rows, z, z, z)
        ms = timed(lambda: part.step(x, ctx))
        active = min(E, n_rows * top) * 2 * eff * width * 2
        note(f"routed_experts_{n_rows}_rows", ms, flops=4.0 * n_rows * top * eff * width, bytes_=active)
    wgu, wd = bf(2 * 18432, width) * 0.05, bf(width, 18432) * 0.05
    for n_rows in (1, 8, 64, T):
        x = bf(n_rows, width)
        ms = timed(lambda: linear(kernels.glu(linear(x, wgu), "gelu_tanh"), wd))
        note(f"dense_gelu_glu_ff_{n_rows}_rows", ms, flops=6.0 * n_rows * 18432 * width, bytes_=3 * 18432 * width * 2)
    kernels.check_bounded_waits(torch.device("cuda", 0))
    print(json.dumps(out))
    return 0


# ---- the Dugopel design beside Fivitar's latent layers and Qwen3 at equal layer sizes -------------------------
def dugopel_config_dict(width, heads, ff, vocab, n_layers, head_dim=128, kv_rank=512, q_rank=1536, rot_dim=64,
                        experts=16, top=2, groups=4, keep=2):
    """`n_layers` layers at sizes of a real model's: a dense feed-forward in the first layer and routed ones (experts
    of ff / top, so that a token's feed-forward has the dense one's parameters) in the others; every third layer
    keeps a latent of its own and the two behind it read its cached rows."""
    def layer(i):
        mixer = {"heads": heads, "dim": head_dim, "rot_dim": rot_dim, "vdim": head_dim, "kv_rank": kv_rank,
                 "q_rank": q_rank, "scale": (head_dim + rot_dim) ** -0.5, "rot": {"base": 10000.0, "dims": rot_dim}}
        if i >= 1 and (i - 1) % 3:
            mixer["kv_from"] = 1 + (i - 1) // 3 * 3
        mlp = {"kind": "dense", "ff": ff, "limit": 7.0} if i == 0 else \
            {"kind": "moe", "expert": {"ff": max(64, ff // top // 64 * 64), "limit": 7.0},
             "router": {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": groups, "keep": keep}}}
        return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}
    return {"architecture": "Dugopel", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "logit_softcap": 30.0, "layers": [layer(i) for i in range(n_layers)]}


def study_dugopel(args, pk) -> int:
    """Prefill (one prompt of 2,048 tokens) and decode (batches of 1, 8 and 64 with 2,048 cached tokens each) of
    Dugopel models with random weights, beside a Fivitar model of latent-attention layers alone and a Qwen3 model of
    the same width, depth, heads and feed-forward parameters, and the design's kernels timed alone beside the
    closest kernels of the other models.  One JSON line."""
    import torch
    from garlic_inference_b200 import LanguageModel, Qwen3Config
    from garlic_inference_b200.config import DugopelConfig, FivitarConfig
    from garlic_inference_b200.ops import counters, glu_product, kernels, linear, swiglu_product
    from garlic_inference_b200.sampling import SamplingParams
    K, W = min(args.steps, 64), max(min(args.warmup, 8), 3)
    torch.cuda.set_device(0)
    greedy = SamplingParams()
    gen = torch.Generator().manual_seed(0)
    sizes = [("1b", 2048, 16, 8192, 32000, 7), ("8b", 4096, 32, 18432, 32000, 4)]
    out = {"study": "dugopel", "dtype": "bfloat16", "data": "synthetic", "steps": K, "warmup": W,
           "peaks": pk, "models": {}, "kernels": {}}

    def timed(fn, reps=5, warm=3):
        for _ in range(warm):
            fn()
        flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda")
        ms = []
        for _ in range(reps):
            flush.zero_()                                  # larger than L2: the next run starts cold
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            ms.append(a.elapsed_time(b))
        return statistics.median(ms)

    def run_model(cfg, vocab):
        per_seq = -(-(CACHED + W + K + 8) // 64) * 64
        model = LanguageModel.from_random(cfg, seed=0, device=0, dtype="bfloat16", max_tokens=64 * per_seq,
                                          max_slots=64)
        eng, sampler = model.engine, model.sampler
        prompt = lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist()
        res = {"weight_bytes": model.model.weight_bytes()}

        def prefill_once():
            s = eng.alloc_slot()
            model.step([(s, prompt(PREFILL_TOKENS), [PREFILL_TOKENS - 1])])
            eng.free_slot(s)
        ms = timed(prefill_once, reps=5, warm=3)
        res["prefill"] = {"tokens": PREFILL_TOKENS, "ms": round(ms, 3), "tokens_per_s": round(PREFILL_TOKENS / ms * 1e3)}
        for batch in (1, 8, 64):
            slots, firsts = [], []
            for _ in range(batch):
                s = eng.alloc_slot()
                firsts.append(sampler.sample(model.step([(s, prompt(CACHED), [CACHED - 1])]), greedy, [0], [0]))
                slots.append(s)
            toks = torch.cat(firsts)
            for _ in range(W):
                toks = sampler.sample(eng.step_decode_device(slots, toks), greedy, slots, slots)
            torch.cuda.synchronize()
            n0 = counters.launches
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(K):
                toks = sampler.sample(eng.step_decode_device(slots, toks), greedy, slots, slots)
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / K
            res[f"decode_b{batch}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(batch / ms * 1e3),
                                       "launches_per_step": (counters.launches - n0) // K}
            for s in slots:
                eng.free_slot(s)
        eng.check()
        del model
        torch.cuda.empty_cache()
        return res

    for label, width, heads, ff, vocab, n_layers in sizes:
        dcfg = DugopelConfig.from_dict(dugopel_config_dict(width, heads, ff, vocab, n_layers))
        fdict = fivitar_config_dict(width, heads, ff * 3 // 2, vocab, 3 * n_layers)      # two matrices: equal parameters
        fdict["layers"] = [l for l in fdict["layers"] if l["type"] == "latent_attention"]
        fcfg = FivitarConfig.from_dict(fdict)
        qcfg = Qwen3Config(hidden_size=width, num_hidden_layers=n_layers, num_attention_heads=heads,
                           num_key_value_heads=max(1, heads // 4), head_dim=128, intermediate_size=ff,
                           vocab_size=vocab, max_position_embeddings=CONTEXT * 2)
        out["models"][label] = {"width": width, "heads": heads, "ff": ff, "layers": n_layers,
                                "dugopel": run_model(dcfg, vocab), "fivitar_latent": run_model(fcfg, vocab),
                                "qwen3": run_model(qcfg, vocab)}

    # ---- the kernels alone, at the larger size: 2,048 rows of a prompt, and 8 single tokens ----
    width, H, d, dr, rank, q_rank, T, page, ffd = 4096, 32, 128, 64, 512, 1536, PREFILL_TOKENS, 64, 18432
    dev = "cuda"
    bf = lambda *shape: torch.randn(*shape, device=dev, dtype=torch.bfloat16) * 0.5
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    kern = out["kernels"]

    def note(name, ms, flops=0.0, bytes_=0.0):
        kern[name] = {"ms": round(ms, 4)}
        if flops:
            kern[name]["tflops"] = round(flops / ms / 1e9, 2)
            kern[name]["of_measured_bf16"] = round(flops / ms / 1e9 / pk["bf16_tflops"], 4)
        if bytes_:
            kern[name]["gbs"] = round(bytes_ / ms / 1e6, 1)
            kern[name]["of_measured_copy"] = round(bytes_ / ms / 1e6 / pk["hbm_gbs"], 3)

    # the norm beside RMSNorm (one and two pending results), the gated unit beside SwiGLU, 2,048 rows and 8 rows
    w = bf(width)
    for n_rows in (T, 8):
        res, d1, d2 = torch.randn(n_rows, width, device=dev), bf(n_rows, width), bf(n_rows, width)
        ms = timed(lambda: kernels.add_layernorm(d1, res, w, None, 1e-6, torch.bfloat16, delta2=d2))
        note(f"add2_layernorm_{n_rows}", ms, bytes_=n_rows * width * (2 + 2 + 4 + 4 + 2))
        ms = timed(lambda: kernels.add_layernorm(d1, res, w, None, 1e-6, torch.bfloat16))
        note(f"add_layernorm_{n_rows}", ms, bytes_=n_rows * width * (2 + 4 + 4 + 2))
        ms = timed(lambda: kernels.add_rmsnorm(d1, res, w, 1e-6, torch.bfloat16))
        note(f"add_rmsnorm_{n_rows}", ms, bytes_=n_rows * width * (2 + 4 + 4 + 2))
        gu = bf(n_rows, 2 * ffd)
        unit = kernels.glu_shape("swish", 1.702, 7.0, 7.0, 1.0)
        ms = timed(lambda: kernels.glu(gu, unit))
        note(f"clamped_swish_glu_{n_rows}", ms, bytes_=n_rows * ffd * 6)
        ms = timed(lambda: kernels.swiglu(gu))
        note(f"swiglu_{n_rows}", ms, bytes_=n_rows * ffd * 6)
        x = bf(n_rows, q_rank + 8)
        ms = timed(lambda: kernels.rmsnorm_rows(x[:, :q_rank], w[:q_rank], 1e-6))
        note(f"rmsnorm_rows_{n_rows}", ms, bytes_=n_rows * q_rank * 4)
    # rotation and cache append in the two layouts; attention over the latent rows is the kernel Fivitar's layers run
    row = rank + dr
    pool = bf(8 * T // page, 1, page, row)
    table = torch.arange(8 * T // page, dtype=torch.int32, device=dev).view(8, T // page)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    freq = torch.tensor([10000.0 ** (-2.0 * i / dr) for i in range(dr // 2)], dtype=torch.float32, device=dev)
    for n_rows, pos, slot in ((T, torch.arange(T, dtype=torch.int32, device=dev), i32([0] * T)),
                              (8, i32([T - 1] * 8), i32(list(range(8))))):
        q_src, kv_src, q_lat = bf(n_rows, H * (d + dr)), bf(n_rows, row), bf(n_rows, H, rank)
        for half in (True, False):
            ms = timed(lambda: kernels.latent_prepare(q_src, 0, kv_src, 0, q_lat, w[:rank], 1e-6, freq, 1.0, dr, pos, slot,
                                                      table, pool, H, d, dr, rank, status, half_layout=half))
            note(f"latent_prepare_{'halves' if half else 'pairs'}_{n_rows}", ms,
                 bytes_=n_rows * (H * (dr + rank) * 2 + row * 2 + H * row * 2 + row * 2))
    q8, pos8, slots8 = bf(8, H, row), i32([T - 1] * 8), i32(list(range(8)))
    ms = timed(lambda: kernels.latent_decode(q8, pool, table, pos8, slots8, 0.07, None, rank, status))
    note("latent_attention_decode_b8", ms, flops=2.0 * 8 * H * (row + rank) * T, bytes_=8 * T * row * 2)
    q, rows = bf(T, H, row), pool.view(-1, page, row)[:T // page].reshape(T, row)

    def by_products():
        for q0 in range(0, T, 1024):
            scores = torch.mm(q[q0:q0 + 1024].view(1024 * H, row), rows[:q0 + 1024].t(), out_dtype=torch.float32)
            wts = kernels.causal_sink_softmax(scores, H, q0, 0.07, None, torch.bfloat16)
            torch.mm(wts, rows[:q0 + 1024, :rank])
    ms = timed(by_products)
    note("latent_attention_prefill2048_products", ms, flops=2.0 * H * (row + rank) * T * (T + 1) / 2)
    # the router beside the other design's, the gated experts beside the two-matrix experts and a dense feed-forward
    from garlic_inference_b200.parts import Runtime, StepContext, part_class
    E, top, eff = 16, 2, ffd // 2
    for n_rows in (8, T):
        z = torch.randn(n_rows, E, device=dev)
        ms = timed(lambda: kernels.router_select(z, top, 4, 2, 2.5))
        note(f"router_select_{n_rows}", ms)
        ms = timed(lambda: kernels.router_topk(z, top))
        note(f"router_topk_{n_rows}", ms)

    def experts_part(gated):
        class Load:
            def dtype(self, *a):
                return torch.bfloat16

            def __call__(self, n, out=None):
                rows_ = eff if gated else eff * 3 // 2
                shape = (E, width) if n == "router" else ((width, rows_) if n.endswith("down") else (rows_, width))
                t = bf(*shape) * 0.05
                return t if out is None else out.copy_(t)
        params = dict(hidden_size=width, expert_size=eff if gated else eff * 3 // 2, n_experts=E, top=top)
        if gated:
            params.update(expert="glu", activation="swish", swish_alpha=1.702, gate_max=7.0, up_limit=7.0, up_shift=1.0,
                          scores="softmax_all", groups=4, groups_kept=2, weight_scale=2.5)
        return part_class("routed_experts")(params, Load(), Runtime(torch.bfloat16, torch.device(dev)))

    zero = i32([0])
    for gated, tag in ((True, "gated_experts"), (False, "two_matrix_experts")):
        part = experts_part(gated)
        for n_rows in (1, 8, 64, T):
            x = bf(n_rows, width)
            ctx = StepContext(n_rows, zero, zero, zero)
            ms = timed(lambda: part.step(x, ctx))
            note(f"{tag}_{n_rows}_rows", ms, flops=6.0 * n_rows * top * eff * width,
                 bytes_=min(E, n_rows * top) * 3 * eff * width * 2)
        del part
        torch.cuda.empty_cache()
    wgu, wd = bf(2 * ffd, width) * 0.05, bf(width, ffd) * 0.05
    unit = kernels.glu_shape("swish", 1.702, 7.0, 7.0, 1.0)
    for n_rows in (1, 8, 64, T):
        x = bf(n_rows, width)
        ms = timed(lambda: linear(glu_product(x, wgu, unit), wd))
        note(f"dense_clamped_swish_ff_{n_rows}_rows", ms, flops=6.0 * n_rows * ffd * width, bytes_=3 * ffd * width * 2)
        ms = timed(lambda: linear(swiglu_product(x, wgu), wd))
        note(f"dense_swiglu_ff_{n_rows}_rows", ms, flops=6.0 * n_rows * ffd * width, bytes_=3 * ffd * width * 2)
    kernels.check_bounded_waits(torch.device("cuda", 0))
    print(json.dumps(out))
    return 0

# ---- the Kenovik design beside Qwen3 at equal layer sizes -------------------------------------------
def kenovik_config_dict(width, heads, ff, vocab, passes, head_dim=128, experts=16, top=2, groups=4, keep=2):
    """Three layers at sizes of a real model's (distance-bias attention + dense, recurrent block + experts, sink
    attention + experts; experts of ff / top, so that a token's routed feed-forward has the dense one's parameters,
    and a shared expert of half that) that run `passes` times in a row."""
    kv = max(1, heads // 4)
    att2 = {"heads": heads, "kv_heads": kv, "dim": head_dim, "vdim": head_dim // 2, "scale": head_dim ** -0.5,
            "bias_max": 2048, "bias_rows": 64, "q_temp": {"coef": 0.1, "every": 512}}
    att = {"heads": heads, "kv_heads": kv, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5,
           "rot": {"base": 500000.0, "dims": head_dim // 2, "scaling": {"factor": 4.0}}}
    rec = {"width": width * 5 // 4, "blocks": max(1, width // 256), "conv": 4}
    eff = max(64, ff // top // 64 * 64)
    moe = {"kind": "moe", "expert": {"ff": eff, "limit": 7.0}, "shared": {"ff": eff // 2, "limit": 7.0},
           "router": {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": groups, "keep": keep}}}
    layers = [{"type": "attention_2", "mixer": att2, "mlp": {"kind": "dense", "ff": ff}},
              {"type": "rglru", "mixer": rec, "mlp": moe}, {"type": "attention", "mixer": att, "mlp": moe}]
    return {"architecture": "Kenovik", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "layers": layers, "loop": {"start": 0, "stop": 3, "times": passes}}


def study_kenovik(args, pk) -> int:
    """Prefill (one prompt of 2,048 tokens) and decode (batches of 1, 8 and 64 with 2,048 cached tokens each) of
    Kenovik models with random weights, beside Qwen3 models of the same width, heads, feed-forward and number of layer
    runs, and the design's kernels timed alone beside the closest kernels of the other models.  One JSON line."""
    import torch
    from garlic_inference_b200 import LanguageModel, Qwen3Config
    from garlic_inference_b200.config import KenovikConfig
    from garlic_inference_b200.ops import counters, kernels
    from garlic_inference_b200.parts import Runtime, StepContext, StepShape, part_class
    from garlic_inference_b200.parts.attention import query_runs
    from garlic_inference_b200.sampling import SamplingParams
    K, W = min(args.steps, 64), max(min(args.warmup, 8), 3)
    torch.cuda.set_device(0)
    greedy = SamplingParams()
    gen = torch.Generator().manual_seed(0)
    sizes = [("1b", 2048, 16, 8192, 32000, 3), ("8b", 4096, 32, 18432, 32000, 2)]
    out = {"study": "kenovik", "dtype": "bfloat16", "data": "synthetic", "steps": K, "warmup": W,
           "peaks": pk, "models": {}, "kernels": {}}

    def timed(fn, reps=5, warm=3):
        for _ in range(warm):
            fn()
        flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda")
        ms = []
        for _ in range(reps):
            flush.zero_()                                  # larger than L2: the next run starts cold
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            ms.append(a.elapsed_time(b))
        return statistics.median(ms)

    def run_model(cfg, vocab):
        per_seq = -(-(CACHED + W + K + 8) // 64) * 64
        model = LanguageModel.from_random(cfg, seed=0, device=0, dtype="bfloat16", max_tokens=64 * per_seq,
                                          max_slots=64)
        eng, sampler = model.engine, model.sampler
        prompt = lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist()
        res = {"weight_bytes": model.model.weight_bytes()}

        def prefill_once():
            s = eng.alloc_slot()
            model.step([(s, prompt(PREFILL_TOKENS), [PREFILL_TOKENS - 1])])
            eng.free_slot(s)
        ms = timed(prefill_once, reps=5, warm=3)
        res["prefill"] = {"tokens": PREFILL_TOKENS, "ms": round(ms, 3), "tokens_per_s": round(PREFILL_TOKENS / ms * 1e3)}
        for batch in (1, 8, 64):
            slots, firsts = [], []
            for _ in range(batch):
                s = eng.alloc_slot()
                firsts.append(sampler.sample(model.step([(s, prompt(CACHED), [CACHED - 1])]), greedy, [0], [0]))
                slots.append(s)
            toks = torch.cat(firsts)
            for _ in range(W):
                toks = sampler.sample(eng.step_decode_device(slots, toks), greedy, slots, slots)
            torch.cuda.synchronize()
            n0 = counters.launches
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(K):
                toks = sampler.sample(eng.step_decode_device(slots, toks), greedy, slots, slots)
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / K
            res[f"decode_b{batch}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(batch / ms * 1e3),
                                       "launches_per_step": (counters.launches - n0) // K}
            for s in slots:
                eng.free_slot(s)
        eng.check()
        del model
        torch.cuda.empty_cache()
        return res

    for label, width, heads, ff, vocab, passes in sizes:
        kcfg = KenovikConfig.from_dict(kenovik_config_dict(width, heads, ff, vocab, passes))
        qcfg = Qwen3Config(hidden_size=width, num_hidden_layers=3 * passes, num_attention_heads=heads,
                           num_key_value_heads=max(1, heads // 4), head_dim=128, intermediate_size=ff,
                           vocab_size=vocab, max_position_embeddings=CONTEXT * 2)
        out["models"][label] = {"width": width, "heads": heads, "ff": ff, "layer_runs": 3 * passes,
                                "kenovik": run_model(kcfg, vocab), "qwen3": run_model(qcfg, vocab)}

    # ---- the kernels alone, at the larger size: 2,048 rows of a prompt, and 8 single tokens ----
    width, H, G, d, T, page, ffd = 4096, 32, 8, 128, PREFILL_TOKENS, 64, 18432
    dev = "cuda"
    bf = lambda *shape: torch.randn(*shape, device=dev, dtype=torch.bfloat16) * 0.5
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    kern = out["kernels"]

    def note(name, ms, flops=0.0, bytes_=0.0):
        kern[name] = {"ms": round(ms, 4)}
        if flops:
            kern[name]["tflops"] = round(flops / ms / 1e9, 2)
            kern[name]["of_measured_bf16"] = round(flops / ms / 1e9 / pk["bf16_tflops"], 4)
        if bytes_:
            kern[name]["gbs"] = round(bytes_ / ms / 1e6, 1)
            kern[name]["of_measured_copy"] = round(bytes_ / ms / 1e6 / pk["hbm_gbs"], 3)

    # the norm that takes a vector along, beside the plain one
    w, off = bf(width), bf(width)
    for n_rows in (T, 8):
        res, d1 = torch.randn(n_rows, width, device=dev), bf(n_rows, width)
        ms = timed(lambda: kernels.add_rmsnorm(d1, res, w, 1e-6, torch.bfloat16, offset=off))
        note(f"add_offset_rmsnorm_{n_rows}", ms, bytes_=n_rows * width * (2 + 4 + 4 + 2))
        ms = timed(lambda: kernels.add_rmsnorm(d1, res, w, 1e-6, torch.bfloat16))
        note(f"add_rmsnorm_{n_rows}", ms, bytes_=n_rows * width * (2 + 4 + 4 + 2))
    # attention: the flash kernel (mma.sync) with a sink, with a distance bias and bare; the tcgen05 kernel bare;
    # the split-KV kernel for 8 single tokens likewise
    table = torch.arange(8 * T // page, dtype=torch.int32, device=dev).view(8, T // page)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    sinks = torch.zeros(H, device=dev)
    dist = torch.randn(2049, H, device=dev)
    runs64 = torch.from_numpy(query_runs(StepShape([0], [0], [T], [0], False), 64)).to(dev)
    runs128 = torch.from_numpy(query_runs(StepShape([0], [0], [T], [0], False), 128)).to(dev)
    pos8, slots8 = i32([T - 1] * 8), i32(list(range(8)))
    for dv, tag in ((128, "k128_v128"), (64, "k128_v64")):
        kp, vp = bf(8 * T // page, G, page, d), bf(8 * T // page, G, page, dv)
        qq, q8 = bf(T, H, d), bf(8, H, d)
        fl = 2.0 * H * (d + dv) * T * (T + 1) / 2
        by = 8 * T * G * (d + dv) * 2
        for name, extra in (("bare", {}), ("sink", {"sinks": sinks}), ("distance_bias", {"dist_bias": dist})):
            ms = timed(lambda: kernels.attention_prefill_masked_bf16(qq, kp, vp, table, runs64, 0.088, rows_covered=True, **extra))
            note(f"attention_prefill2048_mma_{tag}_{name}", ms, flops=fl)
            ms = timed(lambda: kernels.attention_decode_masked_bf16(q8, kp, vp, table, pos8, slots8, 0.088, **extra))
            note(f"attention_decode_b8_mma_{tag}_{name}", ms, bytes_=by)
        if dv == d:
            ms = timed(lambda: kernels.attention_prefill_tcgen05(qq, kp, vp, table, runs128, 0.088, 0, rows_covered=True))
            note(f"attention_prefill2048_tcgen05_{tag}_bare", ms, flops=fl)
            ms = timed(lambda: kernels.attention_prefill_tcgen05(qq, kp, vp, table, runs128, 0.088, 0, rows_covered=True, sinks=sinks))
            note(f"attention_prefill2048_tcgen05_{tag}_sink", ms, flops=fl)
            ms = timed(lambda: kernels.attention_decode_tcgen05(q8, kp, vp, table, pos8, slots8, 0.088, 0))
            note(f"attention_decode_b8_tcgen05_{tag}_bare", ms, bytes_=by)
    # between projections and attention: biases + rotation of half of every head; projection norm + query factor;
    # and Qwen3's kernel (per-head norms, rotation by table)
    freq = torch.tensor([5e5 ** (-2.0 * i / 64) / 4.0 for i in range(32)], dtype=torch.float32, device=dev)
    cols = (H + 2 * G) * d
    bias, wn = torch.randn(cols, device=dev), torch.randn((H + G) * d, device=dev)
    kp, vp = bf(8 * T // page, G, page, d), bf(8 * T // page, G, page, d)
    for n_rows, pos, slot in ((T, torch.arange(T, dtype=torch.int32, device=dev), i32([0] * T)), (8, pos8, slots8)):
        src = bf(n_rows, cols)
        by = n_rows * cols * 2 * 2
        ms = timed(lambda: kernels.attn_prepare(src, 0, H * d, (H + G) * d, freq, 64, False, pos, slot, table, kp, vp, H, d,
                                                torch.bfloat16, status, bias=bias))
        note(f"attn_prepare_bias_rotation_{n_rows}", ms, bytes_=by)
        ms = timed(lambda: kernels.attn_prepare(src, 0, H * d, (H + G) * d, None, 0, False, pos, slot, table, kp, vp, H, d,
                                                torch.bfloat16, status, norm_weight=wn, norm_eps=1e-6, temp_coef=0.1,
                                                temp_every=512))
        note(f"attn_prepare_projection_norm_{n_rows}", ms, bytes_=by)
        ms = timed(lambda: kernels.attn_prepare(src, 0, H * d, (H + G) * d, None, 0, False, pos, slot, table, kp, vp, H, d,
                                                torch.bfloat16, status))
        note(f"attn_prepare_bare_{n_rows}", ms, bytes_=by)
    # the recurrent block's kernels (5,120 channels in 16 blocks, 4 taps) beside the delta rule's scan (16 heads of 128 x 128)
    Wd, B, Kt = 5120, 16, 4
    bw = Wd // B
    taps, xb, cb = bf(Wd, Kt), torch.randn(Wd, device=dev), torch.randn(Wd, device=dev)
    wa, wi = bf(B, bw, bw) * 0.1, bf(B, bw, bw) * 0.1
    ba, bi, lam = torch.randn(Wd, device=dev), torch.randn(Wd, device=dev), torch.randn(Wd, device=dev)
    for n_rows, slot, spans in ((T, i32([0] * T), i32([[0, 0, T]])), (8, slots8, None)):
        proj = bf(n_rows, 2 * Wd)
        state = torch.zeros(9, Kt * Wd, device=dev)
        ms = timed(lambda: kernels.causal_conv_silu(proj[:, Wd:], taps, state[:, Wd:], slot, activation="none", in_bias=xb,
                                                    out_bias=cb, renew_state=spans is None))
        note(f"rglru_conv_{n_rows}", ms, bytes_=n_rows * Wd * (2 + 4))
        u = torch.randn(n_rows, Wd, device=dev)
        ms = timed(lambda: kernels.rglru_gates(u, wa, wi, ba, bi, lam, 8.0))
        note(f"rglru_gates_{n_rows}", ms, flops=4.0 * n_rows * Wd * bw, bytes_=n_rows * Wd * 12 + 2 * B * bw * bw * 2)
        a, b = torch.rand(n_rows, Wd, device=dev), torch.randn(n_rows, Wd, device=dev)
        ms = timed(lambda: kernels.rglru_scan(a, b, proj[:, :Wd], xb, state, spans, slot))
        note(f"rglru_scan_{n_rows}", ms, bytes_=n_rows * Wd * (4 + 4 + 2 + 2))
    Hd, dd = 16, 128
    for n_rows, slot, spans in ((T, i32([0] * T), i32([[0, 0, T]])), (8, slots8, None)):
        qkv = torch.randn(n_rows, 3 * Hd * dd, device=dev)
        ab = torch.randn(n_rows, 2 * Hd, device=dev)
        st = torch.zeros(9, Hd * kernels.scan_state_floats(dd, dd), device=dev)
        A, dt = torch.randn(Hd, device=dev), torch.randn(Hd, device=dev)
        ms = timed(lambda: kernels.delta_scan(qkv, (0, Hd * dd, 2 * Hd * dd), ab, (0, Hd), A, dt, st, spans, slot, Hd, Hd, dd,
                                              dd, 1e-6))
        note(f"delta_scan_{n_rows}", ms, bytes_=n_rows * 3 * Hd * dd * 4 + (2 * 8 * Hd * dd * dd * 4 if spans is None else 0))
    # the router beside the other design's; the gated experts with and without a shared expert
    E, top, eff = 16, 2, ffd // 2
    for n_rows in (8, T):
        z, corr = torch.randn(n_rows, E, device=dev), torch.randn(E, device=dev)
        ms = timed(lambda: kernels.router_select(z, top, 4, 2, 2.5, sigmoid=True, correction=corr, group_top=2, normalize=True))
        note(f"router_sigmoid_corrected_{n_rows}", ms)
        ms = timed(lambda: kernels.router_select(z, top, 4, 2, 2.5))
        note(f"router_softmax_all_{n_rows}", ms)

    def experts_part(shared):
        class Load:
            def dtype(self, *a):
                return torch.bfloat16

            def __call__(self, n, out=None):
                rows_ = eff // 2 if n.startswith("shared") else eff
                shape = (E,) if n == "correction" else (E, width) if n == "router" else \
                    ((width, rows_) if n.endswith("down") else (rows_, width))
                t = bf(*shape) * 0.05
                return t if out is None else out.copy_(t)
        unit = dict(activation="swish", swish_alpha=1.702, gate_max=7.0, up_limit=7.0, up_shift=1.0)
        params = dict(hidden_size=width, expert_size=eff, n_experts=E, top=top, expert="glu", **unit, scores="sigmoid",
                      correction=True, groups=4, groups_kept=2, group_score="top2_sum", normalize=True, weight_scale=2.5)
        if shared:
            params["shared"] = dict(size=eff // 2, **unit)
        return part_class("routed_experts")(params, Load(), Runtime(torch.bfloat16, torch.device(dev)))

    zero = i32([0])
    for shared, tag in ((True, "experts_with_shared"), (False, "experts_alone")):
        part = experts_part(shared)
        for n_rows in (1, 8, 64, T):
            x = bf(n_rows, width)
            ctx = StepContext(n_rows, zero, zero, zero)
            ms = timed(lambda: part.step(x, ctx))
            act = top * eff + (eff // 2 if shared else 0)
            note(f"{tag}_{n_rows}_rows", ms, flops=6.0 * n_rows * act * width,
                 bytes_=(min(E, n_rows * top) * eff + (eff // 2 if shared else 0)) * 3 * width * 2)
        del part
        torch.cuda.empty_cache()
    kernels.check_bounded_waits(torch.device("cuda", 0))
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=32)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration's 36 "
                    "(layer sizes stay); the JSON names both numbers")
    ap.add_argument("--no-points", action="store_true", help="skip decoding at batch 1 and 64")
    ap.add_argument("--write-model", default=None, metavar="DIR",
                    help="with --impl reference: only write the model folder that arm uses (tied head, --layers of the 36) "
                         "to DIR and exit, for running baseline/_ref/bin/reference_runner by hand or under a profiler")
    ap.add_argument("--study", default=None, choices=["prefill-clocks", "fivitar", "zogulorn", "dugopel", "kenovik"],
                    help="prefill-clocks: 40 prompt steps of 2,048 tokens back to back with the clock and the power "
                         "sampled every 20 ms; prints a table and no JSON line.  fivitar: prefill and decode of the "
                         "Fivitar design at two sizes of real layers beside Qwen3 at equal sizes, and the mixers' "
                         "kernels alone; one JSON line of its own.  zogulorn, dugopel, kenovik: the same for those "
                         "designs (dugopel beside Fivitar's latent layers and Qwen3)")
    args = ap.parse_args()

    if args.impl == "reference":
        if args.gpus != 1:
            print(json.dumps({"impl": "reference", "unavailable": "upstream runs on one GPU only"}))
            return 0
        if args.write_model:
            write_reference_model(args.write_model, args.layers or QWEN3_8B["num_hidden_layers"])
            print(f"wrote {args.write_model}")
            return 0
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported (nothing was run)")
        return 2

    if args.study == "fivitar":
        return study_fivitar(args, peaks())
    if args.study == "zogulorn":
        return study_zogulorn(args, peaks())
    if args.study == "dugopel":
        return study_dugopel(args, peaks())
    if args.study == "kenovik":
        return study_kenovik(args, peaks())

    import torch
    from garlic_inference_b200 import LanguageModel, Qwen3Config
    from garlic_inference_b200.ops import counters
    from garlic_inference_b200.sampling import SamplingParams

    K, W = args.steps, max(args.warmup, 3)
    n_layers = args.layers or QWEN3_8B["num_hidden_layers"]
    cfg = Qwen3Config(**{**QWEN3_8B, "num_hidden_layers": n_layers})
    pk = peaks()
    torch.cuda.set_device(0)
    props = torch.cuda.get_device_properties(0)
    gpu_id = "GPU-" + str(props.uuid) if getattr(props, "uuid", None) else "0"
    batches = [args.batch] + ([] if args.no_points else [1, 64])
    per_seq = -(-(CACHED + W + K + 8) // 64) * 64
    long_points = [] if args.no_points else [(8, 8192), (1, 32768)]          # (batch, cached tokens): longer contexts
    max_tokens = max([max(batches) * per_seq, -(-PREFILL_TOKENS // 64) * 64 * 2] +
                     [b * (-(-(c + W + K + 8) // 64) * 64) for b, c in long_points])
    model = LanguageModel.from_random(cfg, seed=0, device=0, dtype="bfloat16", max_tokens=max_tokens)
    eng, sampler = model.engine, model.sampler
    gen = torch.Generator().manual_seed(0)
    greedy = SamplingParams()

    def random_prompt(n):
        return torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()

    def fill(batch, cached=CACHED):
        """`batch` slots, each holding `cached` tokens after a real prefill; returns slots and next tokens."""
        slots, firsts = [], []
        for _ in range(batch):
            s = eng.alloc_slot()
            logits = model.step([(s, random_prompt(cached), [cached - 1])])
            firsts.append(sampler.sample(logits, greedy, [0], [0]))
            slots.append(s)
        return slots, torch.cat(firsts)

    def time_decode(batch, clocks=None, cached=CACHED):
        slots, toks = fill(batch, cached)
        for _ in range(W):
            toks = sampler.sample(eng.step_decode_device(slots, toks), greedy, slots, slots)
        torch.cuda.synchronize()
        launches0 = counters.launches
        if clocks:
            clocks.start()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(K):
            toks = sampler.sample(eng.step_decode_device(slots, toks), greedy, slots, slots)
        end.record()
        torch.cuda.synchronize()
        if clocks:
            clocks.stop()
        ms = start.elapsed_time(end)
        launched = counters.launches - launches0
        for s in slots:
            eng.free_slot(s)
        return batch * K / (ms / 1e3), ms / K, launched

    if args.study == "prefill-clocks":
        return study_prefill_clocks(model, random_prompt(PREFILL_TOKENS), gpu_id,
                                    prefill_flops(QWEN3_8B, n_layers, PREFILL_TOKENS))

    # ---- prefill of 2,048 tokens --------------------------------------------------------------
    prompt = random_prompt(PREFILL_TOKENS)
    times = []
    pre_clocks = ClockSampler(gpu_id, period_ms=20)
    pre_clocks.start()
    for i in range(3 + 5):
        s = eng.alloc_slot()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        model.step([(s, prompt, [PREFILL_TOKENS - 1])])
        b.record()
        torch.cuda.synchronize()
        eng.free_slot(s)
        if i >= 3:
            times.append(a.elapsed_time(b))
    pre_clocks.stop()
    pre_ms = statistics.median(times)
    pre_flops = prefill_flops(QWEN3_8B, n_layers, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (pre_ms / 1e3), "tokens": PREFILL_TOKENS, "ms": pre_ms,
               "frac": pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12),
               "frac_of_sustained": (pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12)
                                     if pk.get("bf16_tflops_sustained") else None),
               "sm_mhz": pre_clocks.summary().get("sm_mhz")}

    # ---- decoding, timed on the device ----------------------------------------------------------
    clocks = ClockSampler(gpu_id)
    value, ms_per_step, launched = time_decode(args.batch, clocks)
    avg_ctx = CACHED + W + (K + 1) / 2
    total_b, weight_b, kv_b = decode_step_bytes(QWEN3_8B, n_layers, args.batch, avg_ctx)
    achieved = total_b / (ms_per_step / 1e3) / 1e9
    points = {}
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = time_decode(b)[0]
        for b, c in long_points:                         # the same through the engine at longer contexts, with the
            tok_s, ms, _ = time_decode(b, cached=c)      # fraction of the measured copy bandwidth the step's bytes reach
            step_b = decode_step_bytes(QWEN3_8B, n_layers, b, c + W + (K + 1) / 2)[0]
            points[f"decode_b{b}_ctx{c}"] = tok_s
            points[f"decode_b{b}_ctx{c}_hbm_frac"] = step_b / (ms / 1e3) / 1e9 / pk["hbm_gbs"]

    # ---- the same through the entry point: host ids in, host ids out, every step ------------------
    # W + K + 1 tokens per request; the clock runs over the last K steps (the W before them are the warm-up,
    # as in the device-timed loop above), read from the loop's own record of when each step's tokens arrived
    prompts = [random_prompt(CACHED) for _ in range(args.batch)]
    model.generate(prompts[:1], max_new_tokens=4)                           # warm the path
    up0 = eng.bytes_uploaded
    e2e_clocks = ClockSampler(gpu_id, period_ms=20)
    wall_minus_perf = time.time() - time.perf_counter()
    e2e_clocks.start()
    out = model.generate(prompts, max_new_tokens=W + K + 1)
    e2e_clocks.stop()
    st = model.last_stats
    assert all(len(o) == W + K + 1 for o in out) and len(st.step_times) == W + K + 1
    e2e_seconds = st.step_times[-1] - st.step_times[-1 - K]
    # the clock during the timed steps of this run (its prompt step of batch x 2,048 tokens comes right before them),
    # so that ms x MHz of the two decode figures can be compared
    e2e_clk = e2e_clocks.summary(since=st.step_times[-1 - K] + wall_minus_perf, until=st.step_times[-1] + wall_minus_perf)
    e2e = {"value": args.batch * K / e2e_seconds, "unit": "tokens/s",
           "h2d_bytes_per_step": (eng.bytes_uploaded - up0) / st.steps,
           "d2h_bytes_per_step": 4 * args.batch, "ms_per_step": 1e3 * e2e_seconds / K,
           "sm_mhz": e2e_clk.get("sm_mhz"), "watts": e2e_clk.get("watts")}
    page_size = eng.cache.page_size
    workloads = {} if args.no_points else larger_workloads(model, pk, gpu_id)

    line = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-8B layer sizes, {CACHED} cached tokens per sequence)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02) made on the GPU, uniform random token ids",
        "config": {"model": "Qwen3-8B layer sizes", "global_batch": args.batch, "seq_len": CONTEXT,
                   "cached_tokens": CACHED, "parallelism": "none (1 GPU)", "layers_run": n_layers,
                   "layers_config": QWEN3_8B["num_hidden_layers"], "hidden_size": 4096, "n_heads": 32,
                   "n_kv_heads": 8, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936,
                   "page_size": page_size, "sampling": "greedy on the device",
                   "l2": "inputs exceed L2: a step reads %.1f GB of weights" % (weight_b / 1e9)},
        "clocks": clocks.summary(),
        "e2e": e2e,
        "gpu_launches": launched,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": total_b, "peaks": pk["source"]},
        "points": points,
        "workloads": workloads,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
