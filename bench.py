"""Benchmark of the engine on one B200: decode and prefill throughput of Qwen2-7B layer sizes
with random weights, with their roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 requests with 1,024-token prompts (the context grows
from 1,024).  ``value`` is decoded tokens a second with the K steps timed on the device;
``e2e`` is the same through the Python entry point (``LLM.step``, with ``overlap``: the next step is
enqueued before the tokens of the one before are read), the step's description going to the device
and the sampled token ids coming to the host every step.  One JSON line is printed.  The engine runs on one GPU: for
--gpus above 1 a line says so and the exit code is 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# layer sizes of Qwen2-7B (v1/models/qwen2-7b/inference_fp16.dag:1-14 of the reference); weights are random, N(0, 0.02)
MODEL = dict(architectures=["Qwen2ForCausalLM"], vocab_size=152064, hidden_size=3584, intermediate_size=18944,
             num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4, head_dim=128, rms_norm_eps=1e-6,
             rope_theta=1000000.0, max_position_embeddings=32768, tie_word_embeddings=False,
             sliding_window=131072, use_sliding_window=False, max_window_layers=28, torch_dtype="bfloat16")
PROMPT_LEN, CONTEXT, PREFILL_TOKENS, PAGE = 1024, 4096, 2048, 64
E2E_SETTLE = 24      # tokens every request decodes between its prompt and the end-to-end run's warm-up steps


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]),
                    bf16_tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def write_reference_weights(folder, model):
    """Random fp16 files with the names and sizes that v1/models/qwen2-7b/inference_fp16.dag:87-142 loads."""
    import torch
    V, H, I, L = model["vocab_size"], model["hidden_size"], model["intermediate_size"], model["num_hidden_layers"]
    KV = model["num_key_value_heads"] * model["head_dim"]
    g = torch.Generator(device="cuda").manual_seed(0)

    def put(name, shape, around_one=False):
        t = torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * 0.02
        if around_one:
            t += 1.0
        t.half().cpu().numpy().tofile(os.path.join(folder, name + ".fp16"))

    put("wte", (V, H))
    put("ln_f", (H,), True)
    put("lm_head", (V, H))
    for i in range(L):
        p = f"h_{i}."
        put(p + "ln_1.weight", (H,), True)
        put(p + "ln_2.weight", (H,), True)
        for proj, rows in (("query", H), ("key", KV), ("value", KV)):
            put(p + f"attn.{proj}.weight", (rows, H))
            put(p + f"attn.{proj}.bias", (rows,))
        put(p + "attn.o_proj.weight", (H, H))
        put(p + "mlp.w1.weight", (I, H))
        put(p + "mlp.w2.weight", (I, H))
        put(p + "mlp.o_proj.weight", (H, I))


def reference_arm(args) -> int:
    """The unmodified vt-transformer v1 engine (its tensor library, CUDA kernels, cuBLASLt and cuDNN calls and its graph
    v1/models/qwen2-7b/inference_fp16.dag), built by baseline/build_reference.sh and driven by baseline/ref_driver.cpp
    as v1/models/qwen2-7b/chat.cpp drives it: the same model sizes, random fp16 weights, 1,024-token prompts, a step
    being one call of its `gpu_main` for the whole batch.  Its step takes the whole token lists from the host and
    gives the sampled ids back to the host, so its figure is an end-to-end one.  MAX_BATCH is set by a second graph
    file, as chat.cpp's command line allows; batch 64 does not fit (its activation buffer for 64 x 4,096 tokens
    alone is 182 GB)."""
    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    if args.gpus != 1:
        return unavailable("vt-transformer's v1 engine runs this model on one GPU")
    driver = os.path.join(REF_DIR, "ref_driver")
    dag = os.path.join(REF_DIR, "src", "models", "qwen2-7b", "inference_fp16.dag")
    if not os.path.isfile(driver) or not os.path.isfile(dag):
        if os.path.isdir(os.path.join(os.environ.get("VT_REFERENCE_CHECKOUT", "/root/reference"), "v1")):
            res = subprocess.run(["bash", os.path.join(ROOT, "baseline", "build_reference.sh")], capture_output=True, text=True)
            if res.returncode != 0:
                return unavailable("baseline/build_reference.sh failed: " + (res.stderr.strip().splitlines() or ["no message"])[-1][:200])
        else:
            return unavailable("baseline/_ref/ref_driver is not built and there is no checkout to build it from "
                               "(baseline/build_reference.sh <checkout>)")
    import shutil
    import tempfile
    import torch
    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    pk = peaks()
    warmup = max(3, args.warmup)
    steps = min(args.steps, 3000 - warmup)               # its cache holds 4,096 tokens a sequence
    # 15 GB of weight files: in memory (/dev/shm) where that has the room, else in the temporary folder
    root, t0 = None, time.time()
    for where in (["/dev/shm"] if os.path.isdir("/dev/shm") else []) + [None]:
        root = tempfile.mkdtemp(prefix="vt_ref_", dir=where)
        try:
            os.makedirs(os.path.join(root, "weights"))
            write_reference_weights(os.path.join(root, "weights"), MODEL)
            break
        except OSError as e:
            shutil.rmtree(root, ignore_errors=True)
            root, why = None, f"the weight files could not be written ({e.__class__.__name__}: {e.strerror})"
    if root is None:
        return unavailable(why)
    try:
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        build_s = time.time() - t0

        def run(batch, k, prefill_runs):
            extra = []
            if batch > 1:
                with open(os.path.join(root, f"batch{batch}.dag"), "w") as f:
                    f.write(f'{batch} "MAX_BATCH" !\n')
                extra = ["--dag", os.path.join(root, f"batch{batch}.dag")]
            cmd = [driver, "--dag", dag, *extra, "--batch", str(batch), "--prompt-len", str(args.prompt_len), "--steps", str(k),
                   "--warmup", str(warmup), "--prefill", str(PREFILL_TOKENS if prefill_runs else 0), "--prefill-runs", str(prefill_runs)]
            res = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=1500)
            lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
            if res.returncode != 0 or not lines:
                raise RuntimeError(f"ref_driver ended with {res.returncode}: {(res.stderr.strip().splitlines() or ['no message'])[-1][:300]}")
            return json.loads(lines[-1])

        clocks = ClockSampler()
        clocks.start()
        try:
            main = run(args.batch, steps, 3)
            info = clocks.stop()
            one = run(1, min(steps, 64), 0) if args.batch != 1 and not args.skip_points else None
        except (RuntimeError, subprocess.TimeoutExpired) as e:
            clocks.stop()
            return unavailable(str(e)[:400])
    finally:
        shutil.rmtree(root, ignore_errors=True)
    cfg = MODEL
    T, H, I, L = PREFILL_TOKENS, cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    q_dim, kv_dim = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    flops = L * (2 * T * H * (q_dim + 2 * kv_dim) + 2 * T * q_dim * H + 6 * T * H * I
                 + 4 * (T * (T + 1) // 2) * cfg["head_dim"] * cfg["num_attention_heads"]) + 2 * H * cfg["vocab_size"]
    pm = main["prefill_ms"]
    ctx_mean = args.prompt_len + warmup + (steps - 1) / 2.0 + 1
    weight_bytes = 2 * (L * (H * (q_dim + 2 * kv_dim) + q_dim + 2 * kv_dim + q_dim * H + 3 * H * I + 2 * H) + H
                        + cfg["vocab_size"] * H + args.batch * H)
    step_bytes = weight_bytes + 2 * 2 * kv_dim * L * ctx_mean * args.batch
    achieved = step_bytes / (main["decode_ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen2-7B layer sizes, random weights, {args.prompt_len:,}-token prompts)",
        "value": round(main["decode_tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(main["decode_ms_per_step"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16", "data": "synthetic", "impl": "reference",
        "config": {"model": "Qwen2-7B sizes, random N(0,0.02)", "layers": L, "layers_full": L, "hidden": H,
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": I, "vocab": cfg["vocab_size"], "global_batch": args.batch, "seq_len": 4096,
                   "prompt_len": args.prompt_len, "mean_context": round(ctx_mean, 1), "parallelism": "1 GPU",
                   "l2": "inputs larger than L2 (every step reads all weights)", "peaks": pk["source"],
                   "timing": "wall clock around whole steps, device idle on both sides",
                   "engine": "vt-transformer v1, inference_fp16.dag, unmodified, MAX_BATCH from a second graph file"},
        "e2e": {"value": round(main["decode_tok_s"], 1), "unit": "tok/s",
                "h2d_bytes_per_step": int(2 * 4 * args.batch * ctx_mean), "d2h_bytes_per_step": 4 * args.batch,
                "note": "the engine's step takes the whole token lists and masks from the host and returns the sampled ids"},
        "clocks": {"sm_mhz": info.get("sm_mhz"), "sm_max_mhz": info.get("sm_max_mhz"), "reasons": info.get("reasons", []),
                   "note": "sampled over the whole run of the engine, its loading of the weights included"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "prefill": {"value": round(T / (pm / 1e3), 1), "tokens": T, "ms": round(pm, 3),
                    "frac": round(flops / (pm / 1e3) / (pk["bf16_tflops"] * 1e12), 4), "tflops": round(flops / pm / 1e9, 1),
                    "ms_all": main["prefill_ms_all"]},
        "points": {"decode_b1": round(one["decode_tok_s"], 1)} if one else {},
        "build_s": round(build_s, 1),
    }
    print(json.dumps(line))
    return 0


# layer sizes of the two smaller models of the family, for the workloads measured beside the headline
MODEL_1_5B = dict(MODEL, hidden_size=1536, intermediate_size=8960, num_attention_heads=12, num_key_value_heads=2,
                  vocab_size=151936, tie_word_embeddings=True, max_window_layers=28)
MODEL_0_5B = dict(MODEL, hidden_size=896, intermediate_size=4864, num_hidden_layers=24, num_attention_heads=14,
                  num_key_value_heads=2, head_dim=64, vocab_size=151936, tie_word_embeddings=True, max_window_layers=24)


def other_points(pk, dev="cuda:0"):
    """Three workloads at the sizes of the family's smaller models (random weights, bfloat16, pages of 64), as flat
    numbers for `points`:

    q15_*: 1.5B sizes, 32 requests at once with prompt lengths uniform in [64, 8192] (seeded) and 128 new tokens
    each, through ``LLM`` with a budget of 2,048 tokens a step: prompt portions beside decoded tokens.
    q05_decode_b256*: 0.5B sizes, decode steps of 256 requests after 512-token prompts, with the step's fraction of
    the HBM roofline.  q05_prefill32k_*: 0.5B sizes, one prompt of 32,768 tokens in portions of 2,048."""
    import random

    import torch
    from vt_transformer_b200 import LLM, SamplingParams, ops
    from vt_transformer_b200.config import config_from_dict
    from vt_transformer_b200.engine import ModelRunner, StepEntry
    out = {}
    gen = torch.Generator().manual_seed(2)

    # ---- 1.5B sizes: 32 concurrent requests, mixed steps
    cfg = config_from_dict(MODEL_1_5B)
    rng = random.Random(7)
    lens = [rng.randint(64, 8192) for _ in range(32)]
    new = 128
    runner = ModelRunner.from_random(cfg, seed=0, sigma=0.02, dtype="bfloat16", device=dev, page_size=PAGE,
                                     num_pages=sum(-(-(n + new + 2) // PAGE) for n in lens) + 8, max_requests=32,
                                     max_seq_len=8192 + new + PAGE)
    best = None
    for rep in range(2):                                    # the first run captures the graphs of its steps
        llm = LLM(None, runner=runner, max_extend_tokens=2048, overlap=True)
        for n in lens:
            llm.add_request(torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist(),
                            SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        produced, mixed, decode = 0, [], []
        while llm.has_work():
            t1 = time.perf_counter()
            res = llm.step()
            dt = (time.perf_counter() - t1) * 1e3
            produced += len(res.results)
            if res.results and res.n_tokens > len(res.results) + 32:
                mixed.append(dt)
            elif res.results:
                decode.append(dt)
        torch.cuda.synchronize()
        el = time.perf_counter() - t0
        if produced != 32 * new:
            raise RuntimeError(f"1.5B workload: {produced} tokens generated, {32 * new} expected")
        best = dict(el=el, mixed=mixed, decode=decode) if best is None or el < best["el"] else best
    out["q15_generated_tok_s"] = round(32 * new / best["el"], 1)
    out["q15_all_tok_s"] = round((sum(lens) + 32 * new) / best["el"], 1)
    out["q15_mixed_step_ms"] = round(statistics.median(best["mixed"]), 3) if best["mixed"] else None
    out["q15_decode_step_ms"] = round(statistics.median(best["decode"]), 3) if best["decode"] else None
    del llm, runner
    torch.cuda.empty_cache()

    # ---- 0.5B sizes: decode steps of 256 requests
    cfg = config_from_dict(MODEL_0_5B)
    B, P, steps, warm = 256, 512, 64, 6
    runner = ModelRunner.from_random(cfg, seed=0, sigma=0.02, dtype="bfloat16", device=dev, page_size=PAGE,
                                     num_pages=B * (P + steps + warm + PAGE) // PAGE + 8, max_requests=B, max_seq_len=1024)
    rows = [runner.admit() for _ in range(B)]
    for i in range(0, B, 4):
        runner.step([StepEntry(r, torch.randint(0, cfg.vocab_size, (P,), generator=gen).tolist(), []) for r in rows[i:i + 4]])
    tok = torch.empty(B, dtype=torch.int32, device=dev)
    feeds = [torch.randint(0, cfg.vocab_size, (B,), generator=gen).tolist() for _ in range(steps + warm)]

    def one(i):
        ops.argmax(runner.step([StepEntry(r, [feeds[i][j]], [0]) for j, r in enumerate(rows)]), tok)

    for i in range(warm):
        one(i)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(warm, warm + steps):
        one(i)
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / steps
    step_bytes = runner.weight_bytes(B) + runner.cache.bytes_per_token() * (P + warm + (steps - 1) / 2.0 + 1) * B
    out["q05_decode_b256"] = round(B / (ms / 1e3), 1)
    out["q05_decode_b256_ms"] = round(ms, 4)
    out["q05_decode_b256_hbm_frac"] = round(step_bytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)
    runner.check_status()
    del runner
    torch.cuda.empty_cache()

    # ---- 0.5B sizes: a prompt of 32,768 tokens in portions of 2,048
    T, C = 32768, 2048
    runner = ModelRunner.from_random(cfg, seed=0, sigma=0.02, dtype="bfloat16", device=dev, page_size=PAGE,
                                     num_pages=T // PAGE + 8, max_requests=2, max_seq_len=T)
    toks = torch.randint(0, cfg.vocab_size, (T,), generator=gen).tolist()
    best = None
    for rep in range(2):
        row = runner.admit()
        times = []
        for a in range(0, T, C):
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            runner.step([StepEntry(row, toks[a:a + C], [C - 1] if a + C == T else [])])
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
        runner.release(row)
        best = times if best is None or sum(times) < sum(best) else best
    runner.check_status()
    H, I, L = cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers
    gemm = L * (2 * T * H * (cfg.q_dim + 2 * cfg.kv_dim) + 2 * T * cfg.q_dim * H + 6 * T * H * I) + 2 * H * cfg.vocab_size
    attn = L * 4 * (T * (T + 1) // 2) * cfg.head_dim * cfg.num_attention_heads
    total = sum(best)
    out["q05_prefill32k_tok_s"] = round(T / (total / 1e3), 1)
    out["q05_prefill32k_tflops"] = round((gemm + attn) / total / 1e9, 1)
    out["q05_prefill32k_last_portion_ms"] = round(best[-1], 3)
    # the last portion: 2,048 tokens over 32,768 keys; its products take what the first portion's take, the rest is attention
    last_attn = L * 4 * (C * (T - C) + C * (C + 1) // 2) * cfg.head_dim * cfg.num_attention_heads
    first_attn = L * 4 * (C * (C + 1) // 2) * cfg.head_dim * cfg.num_attention_heads
    if best[-1] > best[0]:
        out["q05_attention_last_portion_tflops"] = round((last_attn - first_attn) / (best[-1] - best[0]) / 1e9, 1)
    del runner
    torch.cuda.empty_cache()
    return out


# ---- --design: a design's layers at sizes that resemble a served model's, beside the closest Qwen2 model of equal size ----

def _sisetar_config(width, ff, gla, att, delta, chunk, pairs=2):
    """``pairs`` times (a gated-linear-attention layer, a parallel layer with a feed-forward)."""
    layers = []
    for _ in range(pairs):
        layers.append({"type": "gla", "mixer": {"heads": gla[0], "dim": gla[1], "vdim": gla[2], "tau": 16.0}, "mlp": None})
        layers.append({"type": "parallel", "mixer": {
            "left": {"heads": att[0], "kv_heads": att[1], "dim": att[2], "vdim": att[2], "rot": {"dims": att[2] // 2, "base": 1e6},
                     "scale": att[2] ** -0.5, "mask": {"size": chunk}},
            "right": {"heads": delta[0], "dim": delta[1]}, "left_scale": 1.0, "right_scale": 1.0},
            "mlp": {"kind": "dense", "ff": ff}})
    return {"architecture": "Sisetar", "vocab": 32768, "width": width, "layers": layers, "embedding": {"scale": 1.0},
            "logit_scale": 1.0, "logit_softcap": 30.0, "norm": {"eps": 1e-6}}


def _vegilix_config(width, ff, ret, att, window, pairs=2):
    """``pairs`` times (a differential-attention layer, a retention layer), each with 8 experts of which a token uses 2
    beside a shared expert; the three experts a token runs have ``ff`` inner values together.  ``att``: (heads, kv heads,
    head size) of the Qwen2 model of equal size: half as many differential heads with two maps of that size over values
    twice as wide."""
    heads, kv_heads, dim = att[0] // 2, max(1, att[1] // 2), att[2]
    mlp = {"kind": "moe", "router": {"experts": 8, "top": 2}, "expert": {"ff": ff // 3 // 64 * 64}, "shared": {"ff": ff // 3 // 64 * 64}}
    layers = []
    for _ in range(pairs):
        layers.append({"type": "attention", "mixer": {
            "heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": 2 * dim, "diff": 0.3, "scale": dim ** -0.5,
            "rot": {"dims": dim // 2, "base": 1e6, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}},
            "mask": {"size": window, "keep_first": 4}}, "mlp": mlp})
        layers.append({"type": "retention", "mixer": {"heads": ret[0], "dim": ret[1], "vdim": ret[2], "rot": {"dims": ret[1], "base": 1e6},
                                                      "decay": [1.0 - 2.0 ** (-5 - 0.5 * h) for h in range(ret[0])]}, "mlp": mlp})
    return {"architecture": "Vegilix", "vocab": 32768, "width": width, "layers": layers, "norm": {"eps": 1e-6}, "residual_mult": 0.7}


def _geponex_config(width, ff, lig, att, pairs=2):
    """``pairs`` times (a latent-attention layer, a lightning layer): the attention alternates between the plain variant
    (ramped rotation frequencies; 8 clamped experts of which a token uses 2 beside a shared expert, the three experts a
    token runs having ``ff`` inner values together) and the variant with a sink and an output gate (a dense xIELU
    feed-forward of ``ff``); the lightning layers take the experts.  ``att``: (heads, kv heads, head size) of the Qwen2 model
    of equal size: as many heads with that plain part, a rotated part half as wide, a keys' latent of 4 heads' width and
    a queries' latent of 12."""
    heads, dim = att[0], att[2]
    inner = ff // 3 // 64 * 64
    moe = {"kind": "moe", "router": {"experts": 8, "top": 2, "scale": 1.5}, "expert": {"ff": inner, "limit": 7.0},
           "shared": {"ff": inner, "limit": 7.0}}
    layers = []
    for i in range(pairs):
        second = i % 2 == 1
        rot = {"dims": dim // 2, "base": 1e6}
        if not second:
            rot["scaling"] = {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}
        layers.append({"type": "latent_attention_2" if second else "latent_attention", "mixer": {
            "heads": heads, "dim": dim, "rot_dim": dim // 2, "vdim": dim, "q_rank": 12 * dim, "kv_rank": 4 * dim,
            "scale": (1.5 * dim) ** -0.5, "rot": rot}, "mlp": {"kind": "dense", "ff": ff} if second else moe})
        layers.append({"type": "lightning", "mixer": {"heads": lig[0], "dim": lig[1], "vdim": lig[2],
                                                      "decay": [1.0 - 2.0 ** (-5 - 0.5 * h) for h in range(lig[0])]}, "mlp": moe})
    return {"architecture": "Geponex", "vocab": 32768, "width": width, "layers": layers, "norm": {"eps": 1e-6, "groups": 2},
            "postln_alpha": 2.0}


def _fosepel_config(width, ff, mem, att, delta):
    """A layer of each kind and a second attention layer, each with a dense feed-forward of ``ff``: a softmax attention with
    capped scores, a query temperature and learned sinks beside a matrix memory (``mem``: heads, keys' and values' sizes); a
    softmax attention with half of each head rotated (ramped frequencies) and an element-wise gate; a softmax attention with
    a sink of score 0 and a gate a head beside the delta rule with one decay a head (``delta``: heads, head size; half as
    many heads of q and k, values twice as wide, convolutions of 4 taps).  ``att``: (heads, kv heads, head size) of the Qwen2
    model of equal size."""
    heads, kv_heads, dim = att
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5}
    rotary = {"type": "attention", "mlp": {"kind": "dense", "ff": ff}, "mixer": dict(left, rot={
        "dims": dim // 2, "base": 1e6, "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}})}
    layers = [
        {"type": "parallel_2", "mlp": {"kind": "dense", "ff": ff}, "mixer": {
            "left": dict(left, softcap=50.0, q_temp={"coef": 0.1, "every": 1024}),
            "right": {"heads": mem[0], "dim": mem[1], "vdim": mem[2], "gate_cap": 15.0}}},
        rotary,
        {"type": "parallel", "mlp": {"kind": "dense", "ff": ff}, "mixer": {
            "left": dict(left), "right": {"heads": delta[0], "kv_heads": max(1, delta[0] // 2), "dim": delta[1], "vdim": 2 * delta[1], "conv": 4}}},
        rotary,
    ]
    return {"architecture": "Fosepel", "vocab": 32768, "width": width, "layers": layers, "norm": {"eps": 1e-6}, "logit_softcap": 30.0}


DESIGN_SIZES = {
    # name: width, feed-forward, (gla heads, dim, vdim), (attention heads, kv heads, head size), (delta heads, dim), chunk
    "w1024": (1024, 4096, (8, 64, 128), (16, 2, 64), (8, 64), 1024),
    "w4096": (4096, 14336, (16, 128, 256), (32, 8, 128), (16, 128), 2048),
}
DESIGNS = {
    # design: how its configuration is made from a row of DESIGN_SIZES
    "sisetar": lambda width, ff, gla, att, delta, chunk: _sisetar_config(width, ff, gla, att, delta, chunk),
    # (the recurrent layer has the gated linear attention's sizes; the window is the other design's chunk)
    "vegilix": lambda width, ff, gla, att, delta, chunk: _vegilix_config(width, ff, gla, att, chunk),
    "geponex": lambda width, ff, gla, att, delta, chunk: _geponex_config(width, ff, gla, att),
    # (the matrix memory has the gated linear attention's sizes)
    "fosepel": lambda width, ff, gla, att, delta, chunk: _fosepel_config(width, ff, gla, att, delta),
}


def design_points(design: str, sizes, steps: int, warmup: int) -> int:
    """Prefill and decode throughput of ``design`` (random weights, bfloat16, pages of 64) at the sizes of
    ``DESIGN_SIZES``, beside a Qwen2 model of the same width, layer count, feed-forward size and attention heads, and the
    device time of every kernel of one prefill step and one decode step of each (eager, CUDA events around each call;
    the steps that give the throughput run as they are served: prefill eager, decode as captured graphs)."""
    if design not in DESIGNS:
        print(f"bench.py: --design knows {', '.join(sorted(DESIGNS))}, not {design!r}")
        return 2
    import torch
    from vt_transformer_b200 import ops
    from vt_transformer_b200.config import config_from_dict
    from vt_transformer_b200.engine import ModelRunner, StepEntry
    dev, pk = "cuda:0", peaks()
    gen = torch.Generator().manual_seed(4)
    P, CTX, B_LIST = 4096, 1024, (8, 64)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)       # larger than L2: written between timed prefills
    out = {"design": design, "dtype": "bf16", "data": "synthetic", "prefill_tokens": P, "decode_context": CTX,
           "peaks": pk, "l2": "flushed between prefill steps; decode steps read weights and caches larger than L2 at w4096",
           "sizes": {}}

    def timed(fn, reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    def per_kernel(runner, entries):
        """Device time of each of the package's kernels in one eager step, by the name of the op."""
        names = [n for n in ("embedding", "rmsnorm", "layernorm", "polynorm", "head_norm_gate", "gla_scan", "delta_scan",
                             "retention_scan", "gated_delta_scan", "conv_tail_update", "memory_scan", "normed_sum", "add_rows", "route_experts", "route_topk", "token_shift", "latent_prepare", "head_matmul", "attention_latent", "xielu",
                             "gate_clamp", "attention_differential", "attention_prepare", "attention_general", "rope_store", "paged_attention", "rope_attention", "linear",
                             "linear_silu_mul", "linear_to_stream", "logits_scale_cap") if hasattr(ops, n)]
        saved, events = {n: getattr(ops, n) for n in names}, []

        def wrap(name, fn):
            def inner(*a, **k):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                r = fn(*a, **k)
                e1.record()
                events.append((name, e0, e1))
                return r
            return inner
        for n in names:
            setattr(ops, n, wrap(n, saved[n]))
        graphs, runner.use_graphs = runner.use_graphs, False
        try:
            runner.step(entries)
            torch.cuda.synchronize()
        finally:
            runner.use_graphs = graphs
            for n in names:
                setattr(ops, n, saved[n])
        total = {}
        nested = {"linear_to_stream", "linear_silu_mul", "rope_attention"}      # these call other ops of the list
        for name, e0, e1 in events:
            if name in nested:
                continue
            total[name] = total.get(name, 0.0) + e0.elapsed_time(e1) * 1e3
        return {k: round(v, 1) for k, v in sorted(total.items())}

    for size in sizes:
        width, ff, gla, att, delta, chunk = DESIGN_SIZES[size]
        vocab = 32768
        models = {
            design: DESIGNS[design](width, ff, gla, att, delta, chunk),
            "qwen2": dict(architectures=["Qwen2ForCausalLM"], vocab_size=vocab, hidden_size=width, intermediate_size=ff,
                          num_hidden_layers=4, num_attention_heads=att[0], num_key_value_heads=att[1], head_dim=att[2],
                          rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=8192, tie_word_embeddings=True),
        }
        res = {}
        for name, raw in models.items():
            cfg = config_from_dict(raw)
            most = max(B_LIST)
            runner = ModelRunner.from_random(cfg, seed=0, sigma=0.02, dtype="bfloat16", device=dev, page_size=PAGE,
                                             num_pages=(most * (CTX + steps + warmup + 2 * PAGE) + P) // PAGE + 8,
                                             max_requests=most, max_seq_len=8192)
            toks = lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist()
            r = {"weight_bytes": runner.weight_bytes(1)}
            prompt = toks(P)

            def prefill():
                flush.zero_()
                row = runner.admit()
                runner.step([StepEntry(row, prompt, [P - 1])])
                runner.release(row)
            for _ in range(max(3, warmup // 3)):
                prefill()
            flush_ms = timed(flush.zero_, 5)
            ms = timed(prefill, 5) - flush_ms
            r["prefill_ms"], r["prefill_tok_s"] = round(ms, 3), round(P / ms * 1e3, 1)
            row = runner.admit()
            r["prefill_kernels_us"] = per_kernel(runner, [StepEntry(row, prompt, [P - 1])])
            runner.release(row)
            for B in B_LIST:
                rows = [runner.admit() for _ in range(B)]
                for i in range(0, B, 4):
                    runner.step([StepEntry(x, toks(CTX), []) for x in rows[i:i + 4]])
                feed = toks(B)
                one = lambda: runner.step([StepEntry(x, [feed[j]], [0]) for j, x in enumerate(rows)])
                for _ in range(max(3, warmup)):
                    one()
                ms = timed(one, steps)
                r[f"decode_b{B}_ms"], r[f"decode_b{B}_tok_s"] = round(ms, 4), round(B / ms * 1e3, 1)
                r[f"decode_b{B}_hbm_fraction_of_{pk['source']}"] = round(runner.weight_bytes(B) / (ms * 1e-3) / (pk["hbm_gbs"] * 1e9), 3)
                if B == max(B_LIST):
                    r[f"decode_b{B}_kernels_us"] = per_kernel(runner, [StepEntry(x, [feed[j]], [0]) for j, x in enumerate(rows)])
                for x in rows:
                    runner.release(x)
            runner.check_status()
            res[name] = r
            del runner
            torch.cuda.empty_cache()
        out["sizes"][size] = res
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--design", default=None, help="instead of the default workload: prefill and decode throughput of this design "
                    "('sisetar', 'vegilix', 'geponex', 'fosepel') at layer sizes that resemble a served model's, beside a Qwen2 model of equal size")
    ap.add_argument("--design-sizes", default="w1024,w4096", help="which of the sizes of --design to run, with commas between them")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the model has (recorded in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="tokens of every request's prompt (recorded in config)")
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64 and the prefill")
    ap.add_argument("--skip-e2e", action="store_true", help="leave out the run through the Python entry point")
    ap.add_argument("--no-overlap", action="store_true",
                    help="end to end: read a step's tokens before the next step is enqueued (LLM(overlap=False))")
    ap.add_argument("--only-prefill", action="store_true", help="time the 2,048-token prefill only (for profiling)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.design:
        return design_points(args.design, [x for x in args.design_sizes.split(",") if x], min(args.steps, 50), args.warmup)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)

    import torch
    from vt_transformer_b200 import LLM, SamplingParams, ops
    from vt_transformer_b200.config import config_from_dict
    from vt_transformer_b200.engine import ModelRunner, StepEntry

    pk = peaks()
    model = dict(MODEL)
    layers_full = model["num_hidden_layers"]
    if args.layers:
        model["num_hidden_layers"] = args.layers
    cfg = config_from_dict(model)
    dev = "cuda:0"
    max_batch = max(64, args.batch)
    new_tokens = warmup + args.steps + 8
    # end to end the requests' prompts run 2,048 tokens a step beside the decoding of those that are through: the
    # first request decodes that many steps more than the last, and none may end inside the timed steps
    e2e_tokens = new_tokens + (args.batch * args.prompt_len + 2047) // 2048 + 8 + E2E_SETTLE
    prompt_len = args.prompt_len
    context = max(CONTEXT, prompt_len + max(e2e_tokens, 256) + PAGE)
    per_req = prompt_len + max(e2e_tokens, 256) + PAGE
    pool_tokens = max_batch * per_req + PREFILL_TOKENS
    t0 = time.time()
    runner = ModelRunner.from_random(cfg, seed=0, sigma=0.02, dtype="bfloat16", device=dev, page_size=PAGE,
                                     num_pages=-(-pool_tokens // PAGE), max_requests=max_batch, max_seq_len=context)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    gen = torch.Generator().manual_seed(1)
    vocab = cfg.vocab_size

    def random_tokens(n):
        return torch.randint(0, vocab, (n,), generator=gen).tolist()

    def fill(batch):
        """Admits `batch` requests and runs their prompts, 2,048 tokens a step."""
        rows = [runner.admit() for _ in range(batch)]
        chunk = max(1, 2048 // prompt_len)
        for i in range(0, batch, chunk):
            toks = [random_tokens(prompt_len) for _ in rows[i:i + chunk]]
            for at in range(0, prompt_len, 2048):
                runner.step([StepEntry(r, t[at:at + 2048], []) for r, t in zip(rows[i:i + chunk], toks)])
        return rows

    def decode_run(batch, steps, warm, clocks=None):
        rows = fill(batch)
        out = torch.empty(batch, dtype=torch.int32, device=dev)
        feeds = [[random_tokens(batch) for _ in range(steps + warm)]][0]

        def one(i):
            logits = runner.step([StepEntry(r, [feeds[i][j]], [0]) for j, r in enumerate(rows)])
            ops.argmax(logits, out)

        for i in range(warm):
            one(i)
        torch.cuda.synchronize()
        if clocks:
            clocks.start()
        launches0 = ops.launches
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(warm, warm + steps):
            one(i)
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        info = clocks.stop() if clocks else None
        launched = ops.launches - launches0
        ctx_mean = prompt_len + warm + (steps - 1) / 2.0 + 1
        runner.check_status()
        for r in rows:
            runner.release(r)
        return dict(tok_s=batch * steps / (ms / 1e3), ms_per_step=ms / steps, launches=launched, ctx_mean=ctx_mean,
                    clocks=info)

    def prefill_times(warm, timed):
        """One request of 2,048 tokens, one step, logits of the last token: the times of `timed` steps in ms."""
        times = []
        for i in range(warm + timed):
            row = runner.admit()
            toks = random_tokens(PREFILL_TOKENS)
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            runner.step([StepEntry(row, toks, [PREFILL_TOKENS - 1])])
            e.record()
            torch.cuda.synchronize()
            if i >= warm:
                times.append(s.elapsed_time(e))
            runner.release(row)
        runner.check_status()
        return times

    points, prefill, prefill_all = {}, None, []
    T, H, I, L = PREFILL_TOKENS, cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers
    per_layer = 2 * T * H * (cfg.q_dim + 2 * cfg.kv_dim) + 2 * T * cfg.q_dim * H + 2 * T * H * 2 * I + 2 * T * I * H
    attn = 2 * 2 * (T * (T + 1) // 2) * cfg.head_dim * cfg.num_attention_heads
    flops = L * (per_layer + attn) + 2 * H * vocab

    def prefill_record(times):
        """The median of all timed prefill steps.  Steps back to back are a load under which the GPU reaches its
        power cap: `frac` is against the burst peak of the matrix product, `frac_sustained` against the peak of a
        seconds-long loop."""
        ms = statistics.median(times)
        return {"value": round(T / (ms / 1e3), 1), "tokens": T, "ms": round(ms, 3),
                "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4), "tflops": round(flops / ms / 1e9, 1),
                "frac_sustained": round(flops / (ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
                "timed_steps": len(times), "ms_min": round(min(times), 3), "ms_max": round(max(times), 3)}

    if not args.skip_points:
        # the prefill is timed before the decode runs and once more after them; the figure is the median of all
        prefill_all += prefill_times(1, 1) if args.only_prefill else prefill_times(3, 5)
        prefill = prefill_record(prefill_all)

    if args.only_prefill:
        main_run = dict(tok_s=0.0, ms_per_step=1.0, launches=0, ctx_mean=0.0, clocks=None)
        args.skip_e2e = True
    else:
        main_run = decode_run(args.batch, args.steps, warmup, ClockSampler())
    kv_bytes = runner.cache.bytes_per_token() * main_run["ctx_mean"] * args.batch
    step_bytes = runner.weight_bytes(args.batch) + kv_bytes
    achieved = step_bytes / (main_run["ms_per_step"] / 1e3) / 1e9

    e2e_s = produced = h2d = d2h = None
    if not args.skip_e2e:
        # end to end: the Python entry point, token ids in from the host and out to the host every step
        llm = LLM(None, runner=runner, max_extend_tokens=2048, overlap=not args.no_overlap)
        params = SamplingParams(temperature=0.0, max_tokens=e2e_tokens, ignore_eos=True)
        for _ in range(args.batch):
            llm.add_request(random_tokens(prompt_len), params)
        # the prompts run first (compute-bound steps under which the GPU lowers its clocks); the requests then decode
        # E2E_SETTLE tokens before the warm-up steps, so that the timed steps are steady decoding as the device-timed ones are
        while any(len(r.output) < E2E_SETTLE for r in llm.scheduler.running) or llm.scheduler.waiting:
            llm.step()
        for _ in range(warmup):
            llm.step()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        produced = 0
        for _ in range(args.steps):
            produced += len(llm.step().results)
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t1
        if produced != args.batch * args.steps:
            raise RuntimeError(f"end to end: {produced} tokens from {args.steps} steps of {args.batch} requests: a request ended early")
        h2d = llm.h2d_bytes_last_step
        d2h = llm.d2h_bytes_last_step
        for req in list(llm.scheduler.running):
            llm.abort(req.uid)
    if not args.skip_points:
        for b in (() if args.only_prefill else (1, 64)):
            points[f"decode_b{b}"] = round(decode_run(b, min(args.steps, 64), 5)["tok_s"], 1)
        if not args.only_prefill:
            prefill_all += prefill_times(1, 3)
            prefill = prefill_record(prefill_all)
    if args.skip_e2e:
        print(json.dumps({"value": round(main_run["tok_s"], 1), "ms_per_step": round(main_run["ms_per_step"], 4),
                          "points": points, "prefill": prefill, "note": "partial run (--skip-e2e): not a bench line"}))
        return 0
    if not args.skip_points and args.layers is None:
        del llm, runner
        torch.cuda.empty_cache()
        points.update(other_points(pk, dev))

    clocks = main_run["clocks"] or {}
    line = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen2-7B layer sizes, random weights, {prompt_len:,}-token prompts)",
        "value": round(main_run["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": "Qwen2-7B sizes, random N(0,0.02)", "layers": cfg.num_hidden_layers, "layers_full": layers_full,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": args.batch, "seq_len": context, "prompt_len": prompt_len,
                   "mean_context": round(main_run["ctx_mean"], 1),
                   "baseline_mean_context": prompt_len + 128, "page_size": PAGE, "parallelism": "1 GPU",
                   "l2": "inputs larger than L2 (every step reads all weights)", "peaks": pk["source"], "e2e_mode": "step by step" if args.no_overlap else "overlap"},
        "e2e": {"value": round(produced / e2e_s, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": main_run["launches"],
        "clocks": {"sm_mhz": clocks.get("sm_mhz"), "sm_max_mhz": clocks.get("sm_max_mhz"), "reasons": clocks.get("reasons", [])},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "points": points, "build_s": round(build_s, 1),
    }
    if prefill is not None:
        line["prefill"] = prefill
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
