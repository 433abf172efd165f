#!/usr/bin/env python3
"""Headline benchmark: decode tokens per second (and prefill of 2,048 tokens) at the layer
sizes of Qwen2.5-7B with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --arch zolulix [--sizes w2048,w3584] [--prompt 2048] [--batch 8] [--steps K]
    python bench.py --arch mefupel [--sizes w2048,w3584] [--prompt 2048] [--batch 8] [--steps K]
    python bench.py --arch leguvik [--sizes w2048,w3584] [--prompt 2048] [--batch 8] [--steps K]
    python bench.py --arch bulodra [--sizes w2048,w3584] [--prompt 2048] [--batch 8] [--steps K]

Prints ONE JSON line.  (`--arch zolulix` is a measurement of its own: the Zolulix design beside the
Qwen2.5 decoder of equal sizes and its kernels alone; without it the workload below runs.)  A "step" is one decode step of the whole batch.  The default run is a
batch of 8 sequences with 2,048-token prompts in a 4,096-token context; decode at batch 1 and
64 goes into "points".  `value` is timed on the device with CUDA events around K steps of the
engine's decode loop; `e2e` is the same loop driven through the Python entry point with the
step's token ids copied from pinned host memory and the new ids read back every step.
The decode step reads every weight once (14 GB, far above the 126 MB L2), so no L2 flush is
needed between steps; `config` says so.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Layer sizes of Qwen2.5-7B (the benchmark configuration).
QWEN25_7B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=3584,
                 num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4,
                 intermediate_size=18944, vocab_size=152064, rope_theta=1000000.0,
                 rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=False,
                 max_position_embeddings=32768)
PROMPT_LEN, CONTEXT = 2048, 4096
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        def find(d, key):
            """The number under `key`, at the top or one dictionary down."""
            if isinstance(d, dict):
                if isinstance(d.get(key), (int, float)):
                    return float(d[key])
                for v in d.values():
                    if isinstance(v, dict) and isinstance(v.get(key), (int, float)):
                        return float(v[key])
            raise KeyError(key)
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": find(d, "hbm_gbs"), "bf16_tflops": find(d, "bf16_tflops"),
                    "source": "measured"}
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples the SM clock and the throttle reasons (read-only NVML queries) every 50 ms while
    a timed region runs."""
    REASONS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20,
               "hw_thermal_slowdown": 0x40}

    def __init__(self):
        self.samples, self.max_mhz, self._stop, self._thread = [], None, None, None

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
        except Exception:
            return self
        self._stop = threading.Event()

        def poll():
            while not self._stop.is_set():
                try:
                    mhz = int(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                    try:
                        why = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
                    except Exception:
                        why = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                    self.samples.append((mhz, why))
                except Exception:
                    pass
                self._stop.wait(0.05)
        self._thread = threading.Thread(target=poll, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        if self._stop is not None:
            self._stop.set()
            self._thread.join(timeout=2)

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no samples"]}
        mhz = sorted(m for m, _ in self.samples)
        reasons = [n for n, bit in self.REASONS.items() if any(w & bit for _, w in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(self.samples)}


def reference_arm() -> int:
    """The reference is a CMake/C++ project (no Python package): it cannot be installed with
    pip, needs its MLIR submodule and GGUF model files to build, and serves one sequence of
    quantized weights at a time."""
    print(json.dumps({"impl": "reference", "unavailable":
                      "hardenedlinux/SonicBoom has no pip-installable package (pip install of the "
                      "source tree fails: no setup.py/pyproject.toml); its build needs the empty "
                      "third_party/llvm-project submodule and GGUF model files"}))
    return 0


def weight_bytes(model) -> int:
    seen, total = set(), 0
    def add(t):
        nonlocal total
        if t is not None and t.data_ptr() not in seen:
            seen.add(t.data_ptr())
            total += t.numel() * t.element_size()
    for b in model.blocks:
        for part in b.parts:
            for v in vars(part).values():
                if hasattr(v, "data_ptr"):
                    add(v)
    add(model.final_norm.weight)
    add(model.head)                       # the embedding table is read for B rows only
    return total


def decode_flops_per_token(cfg) -> float:
    d, ff = cfg["hidden_size"], cfg["intermediate_size"]
    qw = cfg["num_attention_heads"] * (d // cfg["num_attention_heads"])
    kvw = cfg["num_key_value_heads"] * (d // cfg["num_attention_heads"])
    per_layer = 2 * d * (qw + 2 * kvw) + 2 * qw * d + 2 * d * 2 * ff + 2 * ff * d
    return per_layer * cfg["num_hidden_layers"]


QWEN25_1P5B = dict(QWEN25_7B, hidden_size=1536, num_attention_heads=12, num_key_value_heads=2,
                   intermediate_size=8960, vocab_size=151936, tie_word_embeddings=True)
QWEN25_32B = dict(QWEN25_7B, hidden_size=5120, num_hidden_layers=64, num_attention_heads=40,
                  num_key_value_heads=8, intermediate_size=27648)
REPETITIONS = 3       # timed regions of K steps each; the median is reported


def run(args) -> int:
    import torch
    import sonicboom_b200 as sb
    from sonicboom_b200.engine.decode import DecodeLoop
    from sonicboom_b200 import llm, ops
    from sonicboom_b200.sampling import Sampling

    torch.cuda.set_device(0)
    dev = "cuda:0"
    cfg = dict(QWEN25_7B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    t0 = time.time()
    model = sb.random_model(cfg, seed=0, dtype="bfloat16", device=dev, std=0.02)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    gen = torch.Generator().manual_seed(1)

    def kv_bytes_per_token(m):
        return sum(g.bytes_per_token() for g in sb.Engine(m, max_tokens=64).cache.groups)

    def prompts(n, length=PROMPT_LEN, vocab=None):
        return [torch.randint(0, vocab or cfg["vocab_size"], (length,), generator=gen).tolist()
                for _ in range(n)]

    def decode_point(m, batch, steps, warmup, clocks=None, graph=True, prompt_len=PROMPT_LEN,
                     context=CONTEXT, real_prompt=None, reps=REPETITIONS):
        """Prefills `batch` prompts (8 at a time), then times regions of `steps` steps of the
        decode loop on the device with CUDA events: after `warmup` steps and one untimed region,
        `reps` regions back to back; the median region is the result.
        The sequences decode from prompt_len to context positions; the timed steps are the ones
        around the middle of that stretch.  Instead of decoding every token up to there, the
        sequences' lengths are moved forward (the skipped positions hold zeros in the cache; a
        step reads the same bytes either way).  `real_prompt` < prompt_len prefills only that
        many tokens of each prompt and moves the lengths forward over the rest as well."""
        real = real_prompt or prompt_len
        engine = sb.Engine(m, max_tokens=batch * context, n_slots=batch)
        slots = [engine.open() for _ in range(batch)]
        ps = prompts(batch, real, m.spec.vocab)
        first = []
        for i in range(0, batch, 8):
            lg = engine.step([(s, p, [len(p) - 1]) for s, p in zip(slots[i:i + 8], ps[i:i + 8])])
            first += lg.argmax(dim=-1).tolist()
        room = context - prompt_len
        reps = max(1, min(reps, (room - warmup - 2) // steps - 1))
        total = warmup + (reps + 1) * steps
        skip = max(0, min((context + prompt_len) // 2 - total // 2 - real, context - real - total - 2))
        for s in slots:
            engine.cache.reserve(s, real + skip)
            engine.cache.advance(s, real + skip)
        loop = DecodeLoop(engine, slots, total + 2, use_graph=graph)
        loop.run_device(first, warmup + steps)               # warm-up, and one untimed region
        torch.cuda.synchronize()
        ctx_start = engine.length(slots[0]) + warmup + steps
        if clocks is not None:
            clocks.__enter__()
        times = []
        for _ in range(reps):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            loop.run_device(None, steps)
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end))
        if clocks is not None:
            clocks.__exit__()
        mid = sorted(range(reps), key=lambda i: times[i])[reps // 2]      # the median region
        ms = times[mid]
        launches = loop.launches_per_step * steps
        loop.close()
        for s in slots:
            engine.close(s)
        del engine, loop
        torch.cuda.empty_cache()
        nbytes = weight_bytes(m) + batch * (ctx_start + mid * steps + steps / 2.0) * kv_bytes_per_token(m)
        return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launches,
                "bytes_per_step": nbytes, "frac": nbytes / (ms / steps / 1e3) / 1e9 / pk["hbm_gbs"],
                "repetitions": reps, "all_ms_per_step": [t / steps for t in times]}

    def point_record(r):
        return {"tok_s": round(r["tok_s"], 1), "ms_per_step": round(r["ms_per_step"], 4),
                "bytes_per_step": int(r["bytes_per_step"]), "frac": round(r["frac"], 4)}

    def e2e_point(batch, steps, warmup):
        """The same through the Python entry point: host token ids in, host token ids out.
        generate_batch prefills the prompts and runs the decode loop; every step copies the
        step's ids from pinned host memory and reads the new ids back.  The time between
        the callbacks of token `warmup` and token `warmup + steps` is what is reported."""
        engine = sb.Engine(model, max_tokens=batch * CONTEXT, n_slots=batch)
        stamps = []

        def on_token(i, tok):
            if i == 0:
                stamps.append(time.perf_counter())
            return 0
        # decode from 2,048 up to the same stretch around position 3072 that `value` times
        first = (CONTEXT - PROMPT_LEN) // 2 - steps // 2
        outs = llm.generate_batch(llm.Model(model), prompts(batch), max_tokens=first + steps + 1,
                                  ignore_eos=True, engine=engine, on_token=on_token, max_batch=batch)
        assert all(len(o) == first + steps + 1 for o in outs)
        dt = stamps[first + steps] - stamps[first]
        del engine
        torch.cuda.empty_cache()
        return {"tok_s": batch * steps / dt, "h2d": 4 * batch, "d2h": 4 * batch}

    def session_point(steps, warmup):
        """Batch 1 through llm.Session (`boom_llm_prefill` / `boom_llm_decode`): wall time
        per token of one decode call, after `warmup` tokens."""
        sess = llm.session_new(llm.Model(model), CONTEXT)
        sess.prefill(prompts(1)[0])
        stamps = []
        sess.decode(Sampling(max_tokens=warmup + steps + 1), cb=lambda t: stamps.append(time.perf_counter()) or 0)
        sess.free()
        dt = stamps[warmup + steps] - stamps[warmup]
        del sess
        torch.cuda.empty_cache()
        return {"tok_s": round(steps / dt, 1), "ms_per_step": round(dt / steps * 1e3, 4),
                "positions": f"{PROMPT_LEN}..{PROMPT_LEN + warmup + steps}"}

    if args.only == "decode":
        # a small case for profilers: the decode point alone (with --eager: kernel by kernel)
        r = decode_point(model, args.batch, args.steps, args.warmup, graph=not args.eager, reps=1)
        print(json.dumps({"only": "decode", "layers": cfg["num_hidden_layers"], "batch": args.batch,
                          "ms_per_step": round(r["ms_per_step"], 4), "tok_s": round(r["tok_s"], 1)}))
        return 0

    def prefill_point(m, n_tokens, reps):
        engine = sb.Engine(m, max_tokens=n_tokens, n_slots=1)
        (p,) = prompts(1, n_tokens, m.spec.vocab)
        times = []
        for i in range(1 + reps):
            s = engine.open()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.step([(s, p, [n_tokens - 1])])
            end.record()
            torch.cuda.synchronize()
            engine.close(s)
            if i > 0:
                times.append(start.elapsed_time(end))
        del engine
        torch.cuda.empty_cache()
        return sorted(times)[len(times) // 2]

    def prefill_flops(c, n_tokens):
        hd_ = c["hidden_size"] // c["num_attention_heads"]
        return n_tokens * decode_flops_per_token(c) + \
            c["num_hidden_layers"] * 4 * c["num_attention_heads"] * hd_ * n_tokens * n_tokens / 2 + \
            2 * c["hidden_size"] * c["vocab_size"]

    # prefill of one 2,048-token prompt
    prefill_ms = prefill_point(model, PROMPT_LEN, args.prefill_reps)
    hd = cfg["hidden_size"] // cfg["num_attention_heads"]
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "layers": cfg["num_hidden_layers"], "tokens": PROMPT_LEN,
                          "ms": round(prefill_ms, 3)}))
        return 0

    clocks = ClockSampler()
    main = decode_point(model, args.batch, args.steps, args.warmup, clocks=clocks)
    e2e = e2e_point(args.batch, args.steps, args.warmup)
    points = {}
    for b in (1, 64):
        points[f"decode_b{b}"] = point_record(decode_point(model, b, args.steps, args.warmup))
    if not args.no_extras:
        points["session_decode_b1"] = session_point(min(args.steps, 128), 8)
    ops.check_status()

    if not args.no_extras:
        # Further sizes of the same architecture; they do not enter `value`.
        del model
        torch.cuda.empty_cache()
        # Qwen2.5-1.5B sizes: 64 prompts of 16..1,024 tokens, 256 new tokens each at temperature
        # 0.7, through generate_batch (prefill, sampling and the host loop included)
        m15 = sb.random_model(QWEN25_1P5B, seed=0, dtype="bfloat16", device=dev, std=0.02)
        lens = torch.randint(16, 1025, (64,), generator=gen).tolist()
        ps = [torch.randint(0, QWEN25_1P5B["vocab_size"], (n,), generator=gen).tolist() for n in lens]
        llm.generate_batch(llm.Model(m15), ps[:4], max_tokens=8, ignore_eos=True, temperature=0.7, seed=1)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate_batch(llm.Model(m15), ps, max_tokens=256, ignore_eos=True,
                                  temperature=0.7, seed=1)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        points["qwen2.5-1.5b_generate_64x256_t0.7"] = {
            "tok_s": round(sum(len(o) for o in outs) / dt, 1), "seconds": round(dt, 3),
            "prompt_tokens": sum(lens), "new_tokens": sum(len(o) for o in outs), "layers": 28}
        del m15
        torch.cuda.empty_cache()
        # Qwen2.5-32B sizes: prefill of 8,192 tokens; decode at batch 1 and 16 around position
        # 12,288 of 8,192..16,384 (64 tokens of each prompt are prefilled, the lengths are moved
        # forward over the rest: the cache holds zeros there and a step reads the same bytes)
        c32 = dict(QWEN25_32B)
        if args.layers_32b:
            c32["num_hidden_layers"] = args.layers_32b
        m32 = sb.random_model(c32, seed=0, dtype="bfloat16", device=dev, std=0.02)
        ms32 = prefill_point(m32, 8192, 1)
        rec = {"layers": c32["num_hidden_layers"], "layers_full_model": 64,
               "prefill_8192": {"tok_s": round(8192 / (ms32 / 1e3), 1), "ms": round(ms32, 2),
                                "frac": round(prefill_flops(c32, 8192) / (ms32 / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}}
        for b in (1, 16):
            rec[f"decode_b{b}"] = point_record(decode_point(m32, b, 16, 4, prompt_len=8192, context=16384,
                                                            real_prompt=64))
        points["qwen2.5-32b"] = rec
        del m32
        torch.cuda.empty_cache()
        ops.check_status()

    achieved = main["bytes_per_step"] / (main["ms_per_step"] / 1e3) / 1e9
    out = {
        "metric": "decode tok/s at batch 8 (Qwen2.5-7B sizes, 2,048-token prompts, context 4,096)",
        "value": round(main["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random N(0,0.02) weights, uniform random token ids", "impl": "ours",
        "config": {"model": "Qwen2.5-7B sizes", "layers": cfg["num_hidden_layers"],
                   "layers_full_model": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": hd, "intermediate": cfg["intermediate_size"],
                   "vocab": cfg["vocab_size"], "global_batch": args.batch, "seq_len": CONTEXT,
                   "prompt_len": PROMPT_LEN, "parallelism": "none (1 GPU)",
                   "decode_positions": "timed steps centred on position 3072 of 2048..4096",
                   "l2": "inputs larger than L2 (weights read once per step)",
                   "peaks": pk["source"],
                   "repetitions": f"median of {main['repetitions']} timed regions of {args.steps} steps "
                                  f"after {args.warmup} + {args.steps} untimed steps"},
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tok/s",
                "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": int(main["launches"]),
        "clocks": clocks.summary(),
        "prefill": {"value": round(PROMPT_LEN / (prefill_ms / 1e3), 1), "tokens": PROMPT_LEN,
                    "ms": round(prefill_ms, 3),
                    "frac": round(prefill_flops(cfg, PROMPT_LEN) / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "load_s": round(load_s, 1),
        "build": sb.build_info_line(),
    }
    print(json.dumps(out))
    return 0


# ---------------------------------------------------------------------------- --arch zolulix
def zolulix_config(width, n_layers, ff, vocab, heads, dim, rot_dim, vdim, rank, window, r_heads, r_dim, r_vdim):
    """A Zolulix model of the given layer sizes: recurrence and attention layers alternate, every
    second attention layer reads the cache of the one before it."""
    layers, owner = [], None
    for i in range(n_layers):
        mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
        if i % 2 == 0:
            layers.append({"type": "mlstm", "mlp": mlp,
                           "mixer": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "gate_cap": 15.0}})
            continue
        m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
             "scale": (dim + rot_dim) ** -0.5, "mask": {"size": window}, "rot": {"base": 250000.0, "dims": rot_dim}}
        if owner is not None:
            m["kv_from"], owner = owner, None
        else:
            owner = i
        layers.append({"type": "latent_attention", "mixer": m, "mlp": mlp})
    return {"architecture": "Zolulix", "vocab": vocab, "width": width, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-5}, "layers": layers}


ZOLULIX_SIZES = {
    # name: (Zolulix sizes, the Qwen2.5 configuration of equal width, layers, feed-forward and vocabulary)
    "w2048": (dict(width=2048, n_layers=8, ff=8192, vocab=32768, heads=16, dim=64, rot_dim=32, vdim=64, rank=96,
                   window=1024, r_heads=4, r_dim=128, r_vdim=512),
              dict(QWEN25_7B, hidden_size=2048, num_hidden_layers=8, num_attention_heads=16,
                   num_key_value_heads=2, intermediate_size=8192, vocab_size=32768)),
    "w3584": (dict(width=3584, n_layers=8, ff=18944, vocab=32768, heads=28, dim=96, rot_dim=32, vdim=128, rank=224,
                   window=4096, r_heads=8, r_dim=128, r_vdim=448),
              dict(QWEN25_7B, num_hidden_layers=8, vocab_size=32768)),
}


class ArchBench:
    """What the per-architecture measurements share: a timer over single calls with L2 flushed,
    and the prefill and decode points of one model."""

    def __init__(self):
        import torch
        torch.cuda.set_device(0)
        self.dev, self.pk = "cuda:0", peaks()
        self.gen = torch.Generator().manual_seed(1)
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.dev)      # larger than L2

    def timed(self, fn, reps=5):
        """Median device time (ms) of fn(), L2 flushed before every timed call, after 3 warm-up calls."""
        import torch
        for _ in range(3):
            fn()
        ts = []
        for _ in range(reps):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return sorted(ts)[len(ts) // 2]

    def model_points(self, m, n_prompt, batch, steps, warmup):
        import torch
        import sonicboom_b200 as sb
        from sonicboom_b200.engine.decode import DecodeLoop
        gen, timed = self.gen, self.timed
        vocab = m.spec.vocab
        engine = sb.Engine(m, max_tokens=max(n_prompt, batch * (n_prompt + warmup + 2 * steps + 64)), n_slots=batch)
        p = torch.randint(0, vocab, (n_prompt,), generator=gen).tolist()

        def prefill():
            s = engine.open()
            engine.step([(s, p, [n_prompt - 1])])
            engine.close(s)
        pre_ms = timed(prefill, 3)
        slots = [engine.open() for _ in range(batch)]
        first = []
        for i in range(0, batch, 8):
            lg = engine.step([(s, p, [n_prompt - 1]) for s in slots[i:i + 8]])
            first += lg.argmax(dim=-1).tolist()
        loop = DecodeLoop(engine, slots, warmup + 2 * steps + 2)
        loop.run_device(first, warmup)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        loop.run_device(None, steps)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
        launches = loop.launches_per_step
        loop.close()
        for s in slots:
            engine.close(s)
        del engine, loop
        torch.cuda.empty_cache()
        return {"prefill_tokens": n_prompt, "prefill_ms": round(pre_ms, 3),
                "prefill_tok_s": round(n_prompt / (pre_ms / 1e3), 1), "decode_batch": batch,
                "decode_ms_per_step": round(ms, 4), "decode_tok_s": round(batch / (ms / 1e3), 1),
                "decode_launches_per_step": launches, "weight_bytes": weight_bytes(m)}



def zolulix_kernels(bench, z, rows):
    """Each new kernel alone at `rows` rows with its algorithmic bytes (what it must read and
    write once), and the decoder's like kernels (norm, rotation + cache write)."""
    import torch
    from sonicboom_b200 import ops
    dev, pk, timed = bench.dev, bench.pk, bench.timed
    W, ff = z["width"], z["ff"]
    f32, bf = torch.float32, torch.bfloat16
    out = {}

    def rec(name, ms, nbytes, flops=0):
        out[name] = {"us": round(ms * 1e3, 2), "bytes": int(nbytes),
                     "hbm_frac": round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 3)}
        if flops:
            out[name]["tflops"] = round(flops / (ms / 1e3) / 1e12, 2)
    x, y = torch.randn(rows, W, device=dev), torch.randn(rows, W, device=dev)
    w = torch.ones(W, device=dev, dtype=bf)
    o, nb = torch.empty(rows, W, device=dev), torch.empty(rows, W, device=dev, dtype=bf)
    rec("rmsnorm (decoder's)", timed(lambda: ops.rmsnorm(x, w, 1e-5, nb)), rows * W * 6)
    rec("norm_add + next norm", timed(lambda: ops.norm_add(y, x, w, 1e-5, o, (w, 1e-5, nb))), rows * W * 14)
    n_in = z["n_layers"] // 2 + 1
    planes = torch.randn(n_in, rows, W, device=dev)
    coef = torch.ones(n_in, device=dev, dtype=bf)
    rec(f"depth_mix of {n_in} + next norm", timed(lambda: ops.depth_mix(planes, n_in, coef, o, (w, 1e-5, nb))),
        rows * W * (4 * n_in + 6))
    gu, t = torch.randn(rows, 2 * ff, device=dev), torch.empty(rows, ff, device=dev, dtype=bf)
    rec("glu_clamped", timed(lambda: ops.glu_clamped(gu, 7.0, 1.702, t)), rows * ff * 10)
    H, dim, rd, vd, rank = z["heads"], z["dim"], z["rot_dim"], z["vdim"], z["rank"]
    wide = rank + rd
    proj = torch.randn(rows, H * (dim + rd) + wide, device=dev)
    cache = torch.zeros((rows + 63) // 64, 2, 1, 64, wide, device=dev, dtype=bf)
    q_wide = torch.empty(1, rows, H, wide, device=dev, dtype=bf)
    inv = torch.ones(rd // 2, device=dev)
    row_seq = torch.zeros(rows, dtype=torch.int32, device=dev)
    row_pos = torch.arange(rows, dtype=torch.int32, device=dev)
    page_off = torch.tensor([0, cache.shape[0]], dtype=torch.int32, device=dev)
    page_ids = torch.arange(cache.shape[0], dtype=torch.int32, device=dev)
    cn = torch.ones(rank, device=dev, dtype=bf)
    rec("latent_prep", timed(lambda: ops.latent_prep(proj, H, dim, rd, rank, rd, inv, row_seq, row_pos, page_off,
                                                     page_ids, 64, cn, 1e-5, cache, q_wide)),
        rows * (4 * (H * rd + wide) + 2 * H * rd + 4 * wide))
    hq, hkv, hd = 28, 4, 128
    qkv = torch.randn(rows, (hq + 2 * hkv) * hd, device=dev)
    cache2 = torch.zeros((rows + 63) // 64, 2, hkv, 64, hd, device=dev, dtype=bf)
    q2 = torch.empty(rows, hq, hd, device=dev, dtype=bf)
    inv2 = torch.ones(hd // 2, device=dev)
    rec("rope_store (decoder's)", timed(lambda: ops.rope_store(qkv, hq, hkv, hd, hd, inv2, row_seq, row_pos, page_off,
                                                                page_ids, 64, cache2, q2)),
        rows * (hq + 2 * hkv) * hd * 6)
    ukt = torch.randn(H, rank, dim, device=dev).to(bf)
    uv = torch.randn(H, vd, rank, device=dev).to(bf)
    zz = torch.randn(rows, H * wide, device=dev).to(bf)
    mixed = torch.empty(rows, H * vd, device=dev, dtype=bf)
    rec("head_linear (queries to latent)",
        timed(lambda: ops.head_linear(proj, 0, proj.shape[1], dim + rd, ukt, q_wide, 0, H * wide, wide, rows)),
        rows * H * (4 * dim + 2 * rank) + 2 * H * rank * dim, 2 * rows * H * dim * rank)
    rec("head_linear (latent to values)",
        timed(lambda: ops.head_linear(zz, 0, H * wide, wide, uv, mixed, 0, H * vd, vd, rows)),
        rows * H * (2 * rank + 2 * vd) + 2 * H * rank * vd, 2 * rows * H * vd * rank)
    rh, rdim, rvd = z["r_heads"], z["r_dim"], z["r_vdim"]

    class Plan:
        n_seqs = 1 if rows > 64 else rows
    per = Plan.max_new = rows // Plan.n_seqs
    Plan.seq_row0 = torch.arange(0, rows + 1, per, dtype=torch.int32, device=dev)
    Plan.seq_slot = torch.arange(Plan.n_seqs, dtype=torch.int32, device=dev)
    rproj = torch.randn(rows, 2 * rh * (rdim + rvd + 1), device=dev) * 0.1
    state = torch.zeros(Plan.n_seqs, rh, rvd + 1, (rdim + 4) // 4 * 4, device=dev)
    num, m_row = torch.empty(rows, rh, rvd + 1, device=dev), torch.empty(rows, rh, device=dev)
    bi = torch.zeros(rh, device=dev, dtype=bf)
    rec(f"mlstm_scan ({Plan.n_seqs} sequence(s) of {per})",
        timed(lambda: ops.mlstm_scan(rproj, Plan, rh, rdim, rvd, bi, bi, 15.0, rdim ** -0.5, state, num, m_row)),
        rows * rh * 4 * (2 * rdim + 2 * rvd + 3) + 8 * state.numel(), 4 * rows * rh * rdim * (rvd + 1))
    ro = torch.empty(rows, rh * rvd, device=dev, dtype=bf)
    nw = torch.ones(rh * rvd, device=dev, dtype=bf)
    rec("mlstm_out", timed(lambda: ops.mlstm_out(num, m_row, rproj, rh, rdim, rvd, nw, 1e-5, ro)),
        rows * rh * rvd * 10)
    return out



def run_zolulix(args) -> int:
    """Prefill and decode throughput of Zolulix models at layer sizes of real models (random
    weights), beside the Qwen2.5 decoder of equal width, depth, feed-forward and vocabulary; and
    each new kernel alone with the bytes it must move, beside the like kernel of that decoder."""
    import torch
    import sonicboom_b200 as sb
    from sonicboom_b200 import ops

    bench = ArchBench()
    dev, pk = bench.dev, bench.pk
    model_points = bench.model_points

    def kernels(z, rows):
        return zolulix_kernels(bench, z, rows)

    result = {"arch": "zolulix", "impl": "ours", "dtype": "bf16", "peaks": pk, "sizes": {},
              "data": "synthetic: random N(0,0.02) weights, uniform random token ids",
              "timing": "CUDA events; kernels alone: median of 5 after 3 warm-up calls, L2 flushed "
                        "(256 MB written) before each; models: prefill median of 3, decode one region of K steps"}
    with ClockSampler() as clocks:
        for name, (z, q) in ZOLULIX_SIZES.items():
            if args.sizes and name not in args.sizes.split(","):
                continue
            zc = zolulix_config(**z)
            rec = {"zolulix_config": {k: v for k, v in z.items()}}
            for label, cfg in (("zolulix", zc), ("qwen2.5 (equal width, layers, ff, vocab)", q)):
                m = sb.random_model(cfg, seed=0, dtype="bfloat16", device=dev, std=0.02)
                rec[label] = model_points(m, args.prompt, args.batch, args.steps, args.warmup)
                del m
                torch.cuda.empty_cache()
            rec["kernels_prefill_rows_%d" % args.prompt] = kernels(z, args.prompt)
            rec["kernels_decode_rows_%d" % args.batch] = kernels(z, args.batch)
            result["sizes"][name] = rec
    ops.check_status()
    result["clocks"] = clocks.summary()
    print(json.dumps(result))
    return 0


# ---------------------------------------------------------------------------- --arch mefupel
def mefupel_config(width, n_layers, ff, vocab, heads, kv_heads, dim, window, r_heads, r_dim, r_vdim, rank=16):
    """A Mefupel model of the given layer sizes: attention, attention, gated linear attention and
    the side-by-side layer in turn, every layer with its feed-forward; no loop (the weights are then
    what a step reads, as in the model beside it)."""
    att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
           "mask": {"size": window}, "rot": {"base": 500000.0, "dims": dim}}
    left = dict(att, rot={"base": 20000.0, "dims": dim // 2})
    right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "rot": {"base": 100000.0, "dims": r_dim},
             "decay": [0.9 + 0.099 * (i + 1) / r_heads for i in range(r_heads)]}
    kinds = [("attention", att), ("attention", att),
             ("gla", {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "tau": 12.0, "decay_rank": rank}),
             ("parallel", {"left": left, "right": right})]
    layers = [{"type": kinds[i % 4][0], "mixer": kinds[i % 4][1], "mlp": {"kind": "dense", "ff": ff}}
              for i in range(n_layers)]
    return {"architecture": "Mefupel", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": layers}


MEFUPEL_SIZES = {
    # name: Mefupel sizes; the Zolulix and Qwen2.5 models beside it are ZOLULIX_SIZES[name]
    "w2048": dict(width=2048, n_layers=8, ff=8192, vocab=32768, heads=16, kv_heads=4, dim=128, window=1024,
                  r_heads=8, r_dim=128, r_vdim=256),
    "w3584": dict(width=3584, n_layers=8, ff=18944, vocab=32768, heads=28, kv_heads=4, dim=128, window=4096,
                  r_heads=14, r_dim=128, r_vdim=256),
}


def mefupel_kernels(bench, z, rows):
    """Each kernel that came with Mefupel alone at `rows` rows, with the bytes it must read and
    write once."""
    import torch
    from sonicboom_b200 import ops
    dev, pk, timed = bench.dev, bench.pk, bench.timed
    W, ff = z["width"], z["ff"]
    f32, bf = torch.float32, torch.bfloat16
    out = {}

    def rec(name, ms, nbytes, flops=0):
        out[name] = {"us": round(ms * 1e3, 2), "bytes": int(nbytes),
                     "hbm_frac": round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 3)}
        if flops:
            out[name]["tflops"] = round(flops / (ms / 1e3) / 1e12, 2)
    x, e = torch.randn(rows, W, device=dev), torch.randn(rows, W, device=dev)
    vec = torch.ones(W, device=dev, dtype=bf)
    w = torch.ones(W, device=dev)
    o, nb = torch.empty(rows, W, device=dev), torch.empty(rows, W, device=dev, dtype=bf)
    rec("stream_add + next norm", timed(lambda: ops.stream_add(x, e, vec, o, (w, 1e-6, nb))), rows * W * 14)
    zf, t = torch.randn(rows, ff, device=dev), torch.empty(rows, ff, device=dev, dtype=bf)
    coef = torch.tensor([0.5, 0.3, 0.2, 0.1], device=dev, dtype=bf)
    rec("polynorm", timed(lambda: ops.polynorm(zf, coef, 1e-6, t)), rows * ff * 6)
    H, G, d = z["heads"], z["kv_heads"], z["dim"]
    n_pages = (rows + 63) // 64
    row_seq = torch.zeros(rows, dtype=torch.int32, device=dev)
    row_pos = torch.arange(rows, dtype=torch.int32, device=dev)
    page_off = torch.tensor([0, n_pages], dtype=torch.int32, device=dev)
    page_ids = torch.arange(n_pages, dtype=torch.int32, device=dev)
    cache = torch.zeros(n_pages, 2, G, 64, d, device=dev, dtype=bf)
    q = torch.empty(rows, H, d, device=dev, dtype=bf)
    inv = torch.ones(d // 2, device=dev)
    proj = torch.randn(rows, (H + 2 * G) * d, device=dev)
    rec("attn_prep (rotated values)",
        timed(lambda: ops.attn_prep(proj, 0, H * d, (H + G) * d, H, G, d, d, d, d, True, inv, inv, None, None, 1e-6,
                                    row_seq, row_pos, page_off, page_ids, 64, cache, q)),
        rows * (H + 2 * G) * d * 6)
    proj2 = torch.randn(rows, (H + G) * d, device=dev)
    qn, kn = torch.ones(H * d, device=dev, dtype=bf), torch.ones(G * d, device=dev, dtype=bf)
    rec("attn_prep (norms, keys as values)",
        timed(lambda: ops.attn_prep(proj2, 0, H * d, -1, H, G, d, d, d, d // 2, False, inv, None, qn, kn, 1e-6,
                                    row_seq, row_pos, page_off, page_ids, 64, cache, q)),
        rows * ((H + G) * d * 4 + (H + 2 * G) * d * 2))
    att, back = torch.randn(rows, H * d, device=dev).to(bf), torch.empty(rows, H * d, device=dev, dtype=bf)
    rec("attn_unrotate", timed(lambda: ops.attn_unrotate(att, back, H, d, d, True, inv, row_pos)), rows * H * d * 4)
    rh, rd, rv = z["r_heads"], z["r_dim"], z["r_vdim"]

    class Plan:
        n_seqs = 1 if rows > 64 else rows
    per = rows // Plan.n_seqs
    Plan.seq_row0 = torch.arange(0, rows + 1, per, dtype=torch.int32, device=dev)
    Plan.seq_slot = torch.arange(Plan.n_seqs, dtype=torch.int32, device=dev)
    rproj = torch.randn(rows, 2 * rh * (rd + rv), device=dev) * 0.1
    zl = torch.randn(rows, rh * rd, device=dev)
    rinv = torch.ones(rd // 2, device=dev)
    rec("linrec_prep (decay logits)", timed(lambda: ops.linrec_prep(rproj, 0, rh * rd, rh, rd, rd ** -0.5, 1.0, 0, False,
                                                                    None, row_pos, zl, 1.0 / 16.0)),
        rows * rh * rd * 24)
    rec("linrec_prep (rotation)", timed(lambda: ops.linrec_prep(rproj, 0, rh * rd, rh, rd, 1.0, rd ** -0.5, rd, False,
                                                                rinv, row_pos)), rows * rh * rd * 16)
    decay = torch.rand(rows, rh * rd, device=dev) * 0.1 + 0.9
    state = torch.zeros(Plan.n_seqs, rh, rv, rd, device=dev)
    ro = torch.empty(rows, rh, rv, device=dev)
    scan_bytes = rows * rh * 4 * (3 * rd + 2 * rv) + 8 * state.numel()
    rec(f"linrec_scan, a decay per channel ({Plan.n_seqs} sequence(s) of {per})",
        timed(lambda: ops.linrec_scan(rproj, 0, rh * rd, 2 * rh * rd, Plan, rh, rd, rv, decay, None, state, ro)),
        scan_bytes, 4 * rows * rh * rd * rv)
    hdec = torch.full((rh,), 0.99, device=dev)
    rec(f"linrec_scan, a decay per head ({Plan.n_seqs} sequence(s) of {per})",
        timed(lambda: ops.linrec_scan(rproj, 0, rh * rd, 2 * rh * rd, Plan, rh, rd, rv, None, hdec, state, ro)),
        scan_bytes - rows * rh * rd * 4, 4 * rows * rh * rd * rv)
    mixed = torch.empty(rows, rh * rv, device=dev, dtype=bf)
    nw = torch.ones(rv, device=dev, dtype=bf)
    rec("linrec_out", timed(lambda: ops.linrec_out(ro, rproj, 2 * rh * rd + rh * rv, rh, rv, nw, 1e-6, mixed)),
        rows * rh * rv * 10)
    return out


def run_mefupel(args) -> int:
    """Prefill and decode throughput of Mefupel models at layer sizes of real models (random
    weights) beside the Zolulix and Qwen2.5 models of equal width, depth, feed-forward and
    vocabulary; and each of its kernels alone beside the like kernels of those models."""
    import torch
    import sonicboom_b200 as sb
    from sonicboom_b200 import ops

    bench = ArchBench()
    dev = bench.dev
    result = {"arch": "mefupel", "impl": "ours", "dtype": "bf16", "peaks": bench.pk, "sizes": {},
              "data": "synthetic: random N(0,0.02) weights, uniform random token ids",
              "timing": "CUDA events; kernels alone: median of 5 after 3 warm-up calls, L2 flushed "
                        "(256 MB written) before each; models: prefill median of 3, decode one region of K steps"}
    with ClockSampler() as clocks:
        for name, z in MEFUPEL_SIZES.items():
            if args.sizes and name not in args.sizes.split(","):
                continue
            zz, q = ZOLULIX_SIZES[name]
            rec = {"mefupel_config": dict(z)}
            for label, cfg in (("mefupel", mefupel_config(**z)), ("zolulix (equal width, layers, ff, vocab)", zolulix_config(**zz)),
                               ("qwen2.5 (equal width, layers, ff, vocab)", q)):
                m = sb.random_model(cfg, seed=0, dtype="bfloat16", device=dev, std=0.02)
                rec[label] = bench.model_points(m, args.prompt, args.batch, args.steps, args.warmup)
                del m
                torch.cuda.empty_cache()
            for rows in (args.prompt, args.batch):
                rec["kernels_rows_%d" % rows] = mefupel_kernels(bench, z, rows)
                rec["like_kernels_rows_%d" % rows] = zolulix_kernels(bench, zz, rows)
            result["sizes"][name] = rec
    ops.check_status()
    result["clocks"] = clocks.summary()
    print(json.dumps(result))
    return 0


# ---------------------------------------------------------------------------- --arch leguvik
def leguvik_config(width, n_layers, vocab, heads, kv_heads, dim, window, keep_first, s_heads, s_vdim, s_state,
                   d_heads, d_dim, experts, top, expert_ff, shared_ff, rank=32, taps=4):
    """A Leguvik model of the given layer sizes: delta rule, attention, state space, state space,
    delta rule, attention over the first attention layer's keys, state space, and so on in turn,
    every layer with a mixture of experts and a shared expert, input convolutions and the pair
    embedding."""
    att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "softcap": 30.0,
           "mask": {"size": window, "keep_first": keep_first}}
    kinds = [("general_delta", {"heads": d_heads, "dim": d_dim, "decay_rank": rank}), ("attention", att),
             ("mamba2", {"heads": s_heads, "vdim": s_vdim, "state": s_state, "groups": 1, "norm_groups": 1, "conv": 4}),
             ("mamba2", {"heads": s_heads, "vdim": s_vdim, "state": s_state, "groups": 1, "norm_groups": 1, "conv": 4}),
             ("general_delta", {"heads": d_heads, "dim": d_dim, "decay_rank": rank}),
             ("attention", dict(att, kv_from=1)),
             ("mamba2", {"heads": s_heads, "vdim": s_vdim, "state": s_state, "groups": 1, "norm_groups": 1, "conv": 4})]
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": expert_ff, "limit": 7.0},
           "shared": {"ff": shared_ff, "limit": 7.0}}
    layers = []
    for i in range(n_layers):
        kind, mixer = kinds[i % 7]
        mixer = dict(mixer)
        if "kv_from" in mixer:
            mixer["kv_from"] = i - 4
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Leguvik", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "canon": {"taps": taps},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 36313, "mul_cur": 27191}},
            "logit_softcap": 30.0, "layers": layers}


LEGUVIK_SIZES = {
    # name: Leguvik sizes; the Mefupel model beside it has the same width, depth and vocabulary, its
    # feed-forward as wide as what a Leguvik token uses (top * expert_ff + shared_ff), the same
    # attention heads and window, and recurrent heads of the delta rule's count and size
    "w2048": dict(width=2048, n_layers=7, vocab=32768, heads=16, kv_heads=4, dim=128, window=1024, keep_first=64,
                  s_heads=64, s_vdim=64, s_state=128, d_heads=32, d_dim=64, experts=32, top=4, expert_ff=1024,
                  shared_ff=2048),
    "w3584": dict(width=3584, n_layers=7, vocab=32768, heads=28, kv_heads=4, dim=128, window=4096, keep_first=128,
                  s_heads=112, s_vdim=64, s_state=128, d_heads=56, d_dim=64, experts=64, top=6, expert_ff=1536,
                  shared_ff=3072),
}


def leguvik_kernels(bench, z, rows, context):
    """Each kernel that came with Leguvik alone at `rows` rows (one sequence of `rows` tokens when
    rows > 64, else `rows` sequences that hold `context` tokens each and go on by one), with the
    bytes it must read and write once, and beside each the like kernel of the framework's other
    models at the same sizes."""
    import torch
    from sonicboom_b200 import ops
    from sonicboom_b200.cache.kv import Cache, KVNeed, StateNeed
    from sonicboom_b200.engine.step import StepEntry, StepPlan
    dev, pk, timed = bench.dev, bench.pk, bench.timed
    W = z["width"]
    f32, bf = torch.float32, torch.bfloat16
    out = {}

    def rec(name, ms, nbytes, flops=0):
        out[name] = {"us": round(ms * 1e3, 2), "bytes": int(nbytes),
                     "hbm_frac": round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 3)}
        if flops:
            out[name]["tflops"] = round(flops / (ms / 1e3) / 1e12, 2)
    prompt = rows > 64
    n_seqs, new = (1, rows) if prompt else (rows, 1)
    past = 0 if prompt else context
    H, G, d, win, keep = z["heads"], z["kv_heads"], z["dim"], z["window"], z["keep_first"]
    sh, sv, sn = z["s_heads"], z["s_vdim"], z["s_state"]
    dh, dd = z["d_heads"], z["d_dim"]
    inner, hk = sh * sv, dh * dd
    channels = inner + 2 * sn
    needs = {None: StateNeed((sh, sv, sn)), "conv": StateNeed((3, channels)), "canon": StateNeed((3, W)),
             "delta": StateNeed((dh, dd, dd)), "gla": StateNeed((dh, dd, dd))}
    cache = Cache([KVNeed(G, d, win, keep), KVNeed(G, d, win, 0)], [needs, None], n_seqs * (past + new + 64), bf, dev,
                  n_slots=n_seqs, model_state={"prev_token": StateNeed((), torch.int32)})
    slots = [cache.open() for _ in range(n_seqs)]
    for s in slots:
        if past:
            cache.reserve(s, past)
            cache.advance(s, past)
        cache.reserve(s, past + new)
    toks = torch.randint(0, z["vocab"], (new,), generator=bench.gen).tolist()
    plan = StepPlan(cache, [StepEntry(s, toks, []) for s in slots], dev)
    kind = f"{n_seqs} sequence(s) of {new}" + (f" after {past}" if past else "")
    # rows of the stream
    x = torch.randn(rows, W, device=dev)
    wn = torch.ones(W, device=dev, dtype=bf)
    nf, nb = torch.empty(rows, W, device=dev), torch.empty(rows, W, device=dev, dtype=bf)
    rec("layernorm (float32 rows out)", timed(lambda: ops.layernorm(x, wn, 1e-5, nf)), rows * W * 8)
    rec("like: rmsnorm (bfloat16 rows out)", timed(lambda: ops.rmsnorm(x, wn, 1e-5, nb)), rows * W * 6)
    cw = torch.randn(W, 4, device=dev).to(bf)
    rec("causal_conv, added to its input (4 taps)",
        timed(lambda: ops.causal_conv(nf, 0, W, cw, None, plan, cache.state[(0, "canon")], nb, add_input=True)),
        rows * W * 6)
    table = torch.randn(z["vocab"], W, device=dev).to(bf)
    pair = torch.randn(65522, W, device=dev).to(bf)
    rec("embed_pair", timed(lambda: ops.embed_pair(plan, cache.state[("model", "prev_token")], table, pair, 65521,
                                                   36313, 27191, nf)), rows * W * 8)
    # attention
    g0, store0 = plan.groups[cache.group_of_entry[0]], cache.groups[cache.group_of_entry[0]].entry_storage(0)
    g1, store1 = plan.groups[cache.group_of_entry[1]], cache.groups[cache.group_of_entry[1]].entry_storage(1)
    store0.normal_()
    store1.normal_()
    q = torch.randn(rows, H, d, device=dev).to(bf)
    o = torch.empty(rows, H * d, device=dev, dtype=bf)
    pb = torch.zeros(H, device=dev)
    if prompt:
        keys = sum(min(i + 1, win) + min(keep, max(0, i + 1 - win)) for i in range(rows))
        kv_bytes = rows * G * d * 4
    else:
        keys = rows * (min(past + 1, win) + min(keep, max(0, past + 1 - win)))
        kv_bytes = keys * G * d * 4
    att_bytes, att_flops = kv_bytes + rows * H * d * 4, 4 * keys * H * d
    rec(f"attention_sigmoid ({kind}; window {win}, {keep} first keys kept)",
        timed(lambda: ops.attention_sigmoid(q, o, plan, cache.group_of_entry[0], store0, H, G, d, win, keep,
                                            d ** -0.5, 30.0, pb)), att_bytes, att_flops)
    rec(f"like: attention, softmax ({kind}; window {win})",
        timed(lambda: ops.attention(q, o, plan, cache.group_of_entry[1], store1, H, G, d, win, d ** -0.5)),
        att_bytes, att_flops)
    rec(f"like: attention, softmax, the mma.sync kernels ({kind}; window {win})",
        timed(lambda: ops.attention(q, o, plan, cache.group_of_entry[1], store1, H, G, d, win, d ** -0.5, kernel="mma")),
        att_bytes, att_flops)
    # delta rule
    rank = 32
    dproj = torch.randn(rows, 5 * hk + rank, device=dev) * 0.1
    w2, w0, ab = (torch.randn(hk, rank, device=dev).to(bf), torch.zeros(hk, device=dev, dtype=bf),
                  torch.zeros(hk, device=dev, dtype=bf))
    aux = torch.empty(rows, 3, hk, device=dev)
    rec("delta_prep", timed(lambda: ops.delta_prep(dproj, hk, 4 * hk, 5 * hk, dh, dd, w2, w0, ab, 0.6065, 1e-6, aux)),
        rows * hk * 20)
    do = torch.empty(rows, dh, dd, device=dev)
    dstate = cache.state[(0, "delta")]
    scan_bytes = rows * hk * 4 * 7 + 8 * n_seqs * dh * dd * dd
    rec(f"delta_scan ({kind}; {dh} heads of {dd} x {dd})",
        timed(lambda: ops.delta_scan(dproj, 0, hk, 2 * hk, aux, plan, dh, dd, dstate, do)), scan_bytes,
        10 * rows * dh * dd * dd)
    decay = torch.rand(rows, hk, device=dev) * 0.1 + 0.9
    rec(f"like: linrec_scan, a decay per channel ({kind}; {dh} heads of {dd} x {dd})",
        timed(lambda: ops.linrec_scan(dproj, 0, hk, 2 * hk, plan, dh, dd, dd, decay, None, cache.state[(0, "gla")], do)),
        rows * hk * 4 * 5 + 8 * n_seqs * dh * dd * dd, 6 * rows * dh * dd * dd)
    # state space
    sproj = torch.randn(rows, 2 * inner + 2 * sn + sh, device=dev) * 0.1
    xbc = torch.empty(rows, channels + inner, device=dev)
    scw, scb = torch.randn(channels, 4, device=dev).to(bf), torch.zeros(channels, device=dev, dtype=bf)
    rec("causal_conv with silu (x | B | C, 4 taps)",
        timed(lambda: ops.causal_conv(sproj, inner, channels, scw, scb, plan, cache.state[(0, "conv")], xbc, act="silu")),
        rows * channels * 8)
    dtb, alog, dsk = (torch.zeros(sh, device=dev, dtype=bf), torch.zeros(sh, device=dev, dtype=bf),
                      torch.ones(sh, device=dev, dtype=bf))
    tdec = torch.empty(rows, sh, device=dev)
    rec("ssd_prep", timed(lambda: ops.ssd_prep(sproj, inner + channels, xbc, 0, channels, sh, sv, dtb, alog, tdec)),
        rows * inner * 8)
    so = torch.empty(rows, sh, sv, device=dev)
    rec(f"linrec_scan, a decay per token and head ({kind}; {sh} heads of {sn} x {sv}, keys and queries shared)",
        timed(lambda: ops.linrec_scan(xbc, inner + sn, inner, channels, plan, sh, sn, sv, None, None, cache.state[0], so,
                                      token_decay=tdec, heads_per_qk=sh)),
        rows * 4 * (2 * sn + 2 * inner + sh) + 8 * n_seqs * sh * sv * sn, 6 * rows * sh * sv * sn)
    mixed = torch.empty(rows, inner, device=dev, dtype=bf)
    snw = torch.ones(inner, device=dev, dtype=bf)
    rec("ssd_out", timed(lambda: ops.ssd_out(so, xbc, 0, sproj, 0, sh, sv, 1, dsk, snw, 1e-5, mixed)), rows * inner * 14)
    # experts
    E, top, eff = z["experts"], z["top"], z["expert_ff"]
    h = torch.randn(rows, W, device=dev).to(bf)
    logits = torch.randn(rows, E, generator=bench.gen).to(dev)          # seeded: the same experts are hit every run
    ids, wts = torch.empty(rows, top, dtype=torch.int32, device=dev), torch.empty(rows, top, device=dev)
    rec("moe_route", timed(lambda: ops.moe_route(logits, top, ids, wts)), rows * (E * 4 + top * 8))
    w_up = torch.randn(E, 2, eff, W, device=dev).to(bf) * 0.02
    w_down = torch.randn(E, W, eff, device=dev).to(bf) * 0.02
    used = int(torch.unique(ids).numel())                # experts that some row chose: their weights are what must be read
    moe_bytes = used * 3 * eff * W * 2 + rows * W * 10 + rows * top * (eff * 4 + W * 8)
    moe_flops = 6 * rows * top * eff * W
    rec(f"moe_experts: group, up, down, combine ({E} experts of {eff}, {top} a row)",
        timed(lambda: ops.moe_experts(h, ids, wts, w_up, w_down, 7.0, 1.702, x)), moe_bytes, moe_flops)
    ff = top * eff
    wgu = torch.randn(2 * ff, W, device=dev).to(bf) * 0.02
    wd = torch.randn(W, ff, device=dev).to(bf) * 0.02
    act = torch.empty(rows, ff, device=dev, dtype=bf)

    def dense():
        ops.linear(h, wgu, act, ops.EPI_SWIGLU, gate=(7.0, 1.702))
        ops.linear(act, wd, x, ops.EPI_RESIDUAL, residual=x)
    rec(f"like: dense gated feed-forward of the same {ff} values a row (two products)", timed(dense),
        3 * ff * W * 2 + rows * W * 10 + rows * ff * 4, moe_flops)
    return out


def run_leguvik(args) -> int:
    """Prefill and decode throughput of Leguvik models at layer sizes of real models (random
    weights) beside the Mefupel models of equal width, depth, vocabulary and feed-forward values a
    token; and each of its kernels alone beside the like kernels of the other models."""
    import torch
    import sonicboom_b200 as sb
    from sonicboom_b200 import ops

    bench = ArchBench()
    dev = bench.dev
    result = {"arch": "leguvik", "impl": "ours", "dtype": "bf16", "peaks": bench.pk, "sizes": {},
              "data": "synthetic: random N(0,0.02) weights, uniform random token ids",
              "timing": "CUDA events; kernels alone: median of 5 after 3 warm-up calls, L2 flushed "
                        "(256 MB written) before each; models: prefill median of 3, decode one region of K steps"}
    with ClockSampler() as clocks:
        for name, z in LEGUVIK_SIZES.items():
            if args.sizes and name not in args.sizes.split(","):
                continue
            mz = dict(width=z["width"], n_layers=z["n_layers"], ff=z["top"] * z["expert_ff"] + z["shared_ff"],
                      vocab=z["vocab"], heads=z["heads"], kv_heads=z["kv_heads"], dim=z["dim"], window=z["window"],
                      r_heads=z["d_heads"], r_dim=z["d_dim"], r_vdim=z["d_dim"])
            rec = {"leguvik_config": dict(z)}
            for label, cfg in (("leguvik", leguvik_config(**z)),
                               ("mefupel (equal width, layers, vocab, feed-forward values a token)", mefupel_config(**mz))):
                m = sb.random_model(cfg, seed=0, dtype="bfloat16", device=dev, std=0.02)
                rec[label] = bench.model_points(m, args.prompt, args.batch, args.steps, args.warmup)
                del m
                torch.cuda.empty_cache()
            for rows in (args.prompt, args.batch):
                rec["kernels_rows_%d" % rows] = leguvik_kernels(bench, z, rows, args.prompt)
            result["sizes"][name] = rec
    ops.check_status()
    result["clocks"] = clocks.summary()
    print(json.dumps(result))
    return 0

# ---------------------------------------------------------------------------- --arch bulodra
def bulodra_config(width, n_layers, vocab, heads, kv_heads, dim, window, l_dim, l_rot, l_vdim, kv_rank, q_rank,
                   experts, top, groups, expert_ff, shared_ff, dense_ff):
    """A Bulodra model of the given layer sizes: attention over a latent, two capped attentions in a
    window, one attention with a sink, and so on in turn; the first layer with a dense feed-forward,
    the others with a mixture of experts in groups and a shared expert."""
    yarn = {"factor": 4.0, "original": 4096, "fast": 16.0, "slow": 2.0}
    kinds = [("latent_attention", {"heads": heads, "dim": l_dim, "rot_dim": l_rot, "vdim": l_vdim, "kv_rank": kv_rank,
                                   "q_rank": q_rank, "scale": (l_dim + l_rot) ** -0.5,
                                   "rot": {"base": 1e5, "dims": l_rot, "scaling": yarn}}),
             ("attention_2", {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                              "softcap": 50.0, "mask": {"size": window}, "rot": {"base": 1e4, "dims": dim // 2}}),
             ("attention_2", {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                              "softcap": 50.0, "mask": {"size": window}, "rot": {"base": 1e4, "dims": dim // 2}}),
             ("attention", {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                            "rot": {"base": 1e4, "dims": dim, "scaling": yarn}})]
    moe = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": 2.0,
                                     "groups": {"count": groups[0], "keep": groups[1]}},
           "expert": {"ff": expert_ff, "limit": 7.0}, "shared": {"ff": shared_ff, "limit": 7.0}}
    layers = [{"type": kinds[i % 4][0], "mixer": kinds[i % 4][1],
               "mlp": {"kind": "dense", "ff": dense_ff} if i == 0 else moe} for i in range(n_layers)]
    return {"architecture": "Bulodra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "residual_mult": 0.6,
            "logit_scale": 0.5, "embedding": {"bigram": {"buckets": 65521, "mul_prev": 36313, "mul_cur": 27191}},
            "layers": layers}


BULODRA_SIZES = {
    # name: Bulodra sizes; the Leguvik model beside it (the closest design: a mixture of clamped gated
    # experts with a shared expert, windowed attention with a score cap, the pair embedding) has the
    # same width, depth, vocabulary, attention heads and window, experts, choices and expert sizes
    "w2048": dict(width=2048, n_layers=8, vocab=32768, heads=16, kv_heads=4, dim=128, window=1024, l_dim=64, l_rot=32,
                  l_vdim=64, kv_rank=96, q_rank=512, experts=32, top=4, groups=(4, 2), expert_ff=1024, shared_ff=2048,
                  dense_ff=8192),
    "w3584": dict(width=3584, n_layers=8, vocab=32768, heads=28, kv_heads=4, dim=128, window=4096, l_dim=96, l_rot=32,
                  l_vdim=128, kv_rank=224, q_rank=768, experts=64, top=6, groups=(8, 4), expert_ff=1536, shared_ff=3072,
                  dense_ff=18944),
}


def bulodra_kernels(bench, z, rows, context):
    """Each kernel that came with Bulodra (or was extended for it) alone at `rows` rows (one sequence
    of `rows` tokens when rows > 64, else `rows` sequences that hold `context` tokens each and go on
    by one), with the bytes it must read and write once, and beside each the like kernel of the
    framework's other models at the same sizes."""
    import torch
    from sonicboom_b200 import ops
    from sonicboom_b200.cache.kv import Cache, KVNeed
    from sonicboom_b200.engine.step import StepEntry, StepPlan
    from sonicboom_b200.parts.rotary import frequency_table
    dev, pk, timed = bench.dev, bench.pk, bench.timed
    W = z["width"]
    f32, bf = torch.float32, torch.bfloat16
    out = {}

    def rec(name, ms, nbytes, flops=0):
        out[name] = {"us": round(ms * 1e3, 2), "bytes": int(nbytes),
                     "hbm_frac": round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 3)}
        if flops:
            out[name]["tflops"] = round(flops / (ms / 1e3) / 1e12, 2)
    prompt = rows > 64
    n_seqs, new = (1, rows) if prompt else (rows, 1)
    past = 0 if prompt else context
    H, G, d, win = z["heads"], z["kv_heads"], z["dim"], z["window"]
    ld, lr, lv, rank, qr = z["l_dim"], z["l_rot"], z["l_vdim"], z["kv_rank"], z["q_rank"]
    wide = rank + lr
    cache = Cache([KVNeed(G, d, win), KVNeed(1, wide, 0)], [None, None], n_seqs * (past + new + 64), bf, dev,
                  n_slots=n_seqs)
    slots = [cache.open() for _ in range(n_seqs)]
    for s in slots:
        if past:
            cache.reserve(s, past)
            cache.advance(s, past)
        cache.reserve(s, past + new)
    plan = StepPlan(cache, [StepEntry(s, [0] * new, []) for s in slots], dev)
    kind = f"{n_seqs} sequence(s) of {new}" + (f" after {past}" if past else "")
    # rows of the stream
    x, y = torch.randn(rows, W, device=dev), torch.randn(rows, W, device=dev)
    wn = torch.ones(W, device=dev)
    wb = torch.ones(W, device=dev, dtype=bf)
    xo, nb = torch.empty(rows, W, device=dev), torch.empty(rows, W, device=dev, dtype=bf)
    rec("norm_add + the stream in bfloat16", timed(lambda: ops.norm_add(y, x, wn, 1e-6, xo, (None, 0.0, nb))), rows * W * 14)
    rec("like: norm_add + next norm", timed(lambda: ops.norm_add(y, x, wn, 1e-6, xo, (wb, 1e-6, nb))), rows * W * 14)
    # queries and cache rows
    g0, store0 = plan.groups[cache.group_of_entry[0]], cache.groups[cache.group_of_entry[0]].entry_storage(0)
    g1, store1 = plan.groups[cache.group_of_entry[1]], cache.groups[cache.group_of_entry[1]].entry_storage(1)
    store0.normal_()
    store1.normal_()
    n_in = (H + 2 * G) * d + H
    proj = torch.randn(rows, n_in, device=dev)
    q = torch.empty(rows, H, d, device=dev, dtype=bf)
    table = frequency_table(1e4, d, dev)
    hw, kw = torch.ones(d, device=dev, dtype=bf), torch.ones(d, device=dev, dtype=bf)
    prep_bytes = rows * ((H + 2 * G) * d * 4 + (H + 2 * G) * d * 2)

    def prep(head_norm, qn, kn, rot):
        return lambda: ops.attn_prep(proj, 0, H * d + H, H * d + H + G * d, H, G, d, d, d, rot, False, table, None, qn, kn,
                                     1e-6, plan.row_seq, plan.row_pos, g0.page_off, g0.page_ids, g0.page_size, store0,
                                     q, head_norm=head_norm, rot_scale=1.2)
    rec("attn_prep, every head normed before the rotation", timed(prep("before", hw, kw, d)), prep_bytes)
    rec("attn_prep, every head normed after the rotation", timed(prep("after", None, None, d // 2)), prep_bytes)
    qn_all, kn_all = torch.ones(H * d, device=dev, dtype=bf), torch.ones(G * d, device=dev, dtype=bf)
    rec("like: attn_prep, the whole projection normed", timed(prep(None, qn_all, kn_all, d)), prep_bytes)
    rec("like: attn_prep, no norm", timed(prep(None, None, None, d)), prep_bytes)
    # attention with a score cap
    o = torch.empty(rows, H * d, device=dev, dtype=bf)
    if prompt:
        keys = sum(min(i + 1, win) for i in range(rows))
        kv_bytes = rows * G * d * 4
    else:
        keys = rows * min(past + 1, win)
        kv_bytes = keys * G * d * 4
    att_bytes, att_flops = kv_bytes + rows * H * d * 4, 4 * keys * H * d
    grp0 = cache.group_of_entry[0]
    rec(f"attention, capped scores ({kind}; window {win})",
        timed(lambda: ops.attention(q, o, plan, grp0, store0, H, G, d, win, d ** -0.5, softcap=50.0)), att_bytes, att_flops)
    rec(f"like: attention ({kind}; window {win})",
        timed(lambda: ops.attention(q, o, plan, grp0, store0, H, G, d, win, d ** -0.5)), att_bytes, att_flops)
    sink = torch.zeros(H, device=dev)
    rec(f"like: attention with a sink ({kind}; window {win})",
        timed(lambda: ops.attention(q, o, plan, grp0, store0, H, G, d, win, d ** -0.5, sink=sink)), att_bytes, att_flops)
    # the gate on every head's result
    og = torch.empty(rows, H * d, device=dev, dtype=bf)
    rec("attn_unrotate with the heads' gates", timed(lambda: ops.attn_unrotate(o, og, H, d, d, False, None, plan.row_pos,
                                                                               gate=(proj, H * d))), rows * H * d * 4)
    o_pad = torch.empty(rows, H * (d + 16), device=dev, dtype=bf)
    rec("like: attn_unrotate (padding dropped)", timed(lambda: ops.attn_unrotate(o_pad, og, H, d + 16, d, False, None,
                                                                                plan.row_pos)), rows * H * d * 4)
    # the latent's rows
    first = torch.randn(rows, qr + wide, device=dev)
    cq = torch.empty(rows, qr, device=dev, dtype=bf)
    wq = torch.ones(qr, device=dev, dtype=bf)
    rec("rmsnorm of a row's first values (the query latent)", timed(lambda: ops.rmsnorm(first, wq, 1e-6, cq, width=qr)),
        rows * qr * 6)
    flat = torch.randn(rows, qr, device=dev)
    rec("like: rmsnorm", timed(lambda: ops.rmsnorm(flat, wq, 1e-6, cq)), rows * qr * 6)
    lproj = torch.randn(rows, H * (ld + lr), device=dev)
    qwide = torch.empty(1, rows, H, wide, device=dev, dtype=bf)
    cn = torch.ones(rank, device=dev, dtype=bf)
    ltab = frequency_table(1e5, lr, dev)
    lbytes = rows * (H * lr * 6 + wide * 4 + wide * 4)
    rec("latent_prep, pairs half the part apart, the latent in rows of its own",
        timed(lambda: ops.latent_prep(lproj, H, ld, lr, rank, lr, ltab, plan.row_seq, plan.row_pos, g1.page_off, g1.page_ids,
                                      g1.page_size, cn, 1e-6, store1, qwide, H, kv=(first, qr), interleaved=False,
                                      rot_scale=1.2)), lbytes)
    lboth = torch.randn(rows, H * (ld + lr) + wide, device=dev)
    rec("like: latent_prep, interleaved pairs, one row",
        timed(lambda: ops.latent_prep(lboth, H, ld, lr, rank, lr, ltab, plan.row_seq, plan.row_pos, g1.page_off, g1.page_ids,
                                      g1.page_size, cn, 1e-6, store1, qwide, H)), lbytes)
    # the router and the dense feed-forward's gate
    E, top = z["experts"], z["top"]
    logits = torch.randn(rows, E, generator=bench.gen).to(dev)
    corr = torch.zeros(E, device=dev)
    ids, wts = torch.empty(rows, top, dtype=torch.int32, device=dev), torch.empty(rows, top, device=dev)
    rec("moe_route_scored (groups)", timed(lambda: ops.moe_route_scored(logits, corr, top, ids, wts, groups=z["groups"],
                                                                        scale=2.0)), rows * (E * 4 + top * 8))
    rec("like: moe_route", timed(lambda: ops.moe_route(logits, top, ids, wts)), rows * (E * 4 + top * 8))
    ff = z["dense_ff"]
    h = torch.randn(rows, W, device=dev).to(bf)
    wgu = torch.randn(2 * ff, W, device=dev).to(bf) * 0.02
    act = torch.empty(rows, ff, device=dev, dtype=bf)
    gu_bytes, gu_flops = 2 * ff * W * 2 + rows * (W + ff) * 2, 4 * rows * ff * W
    rec("gate | up product with gelu in its epilogue", timed(lambda: ops.linear(h, wgu, act, ops.EPI_SWIGLU,
                                                                                gate_kind=ops.GATE_GELU_TANH)), gu_bytes, gu_flops)
    rec("like: gate | up product with silu in its epilogue", timed(lambda: ops.linear(h, wgu, act, ops.EPI_SWIGLU)),
        gu_bytes, gu_flops)
    rec("like: gate | up product with the clamped form in its epilogue",
        timed(lambda: ops.linear(h, wgu, act, ops.EPI_SWIGLU, gate=(7.0, 1.702))), gu_bytes, gu_flops)
    return out


def run_bulodra(args) -> int:
    """Prefill and decode throughput of Bulodra models at layer sizes of real models (random
    weights) beside the Leguvik models of equal width, depth, vocabulary, attention and experts; and
    each of its kernels alone beside the like kernels of the other models."""
    import torch
    import sonicboom_b200 as sb
    from sonicboom_b200 import ops

    bench = ArchBench()
    dev = bench.dev
    result = {"arch": "bulodra", "impl": "ours", "dtype": "bf16", "peaks": bench.pk, "sizes": {},
              "data": "synthetic: random N(0,0.02) weights, uniform random token ids",
              "timing": "CUDA events; kernels alone: median of 5 after 3 warm-up calls, L2 flushed "
                        "(256 MB written) before each; models: prefill median of 3, decode one region of K steps"}
    with ClockSampler() as clocks:
        for name, z in BULODRA_SIZES.items():
            if args.sizes and name not in args.sizes.split(","):
                continue
            lz = dict(width=z["width"], n_layers=z["n_layers"] - 1, vocab=z["vocab"], heads=z["heads"],
                      kv_heads=z["kv_heads"], dim=z["dim"], window=z["window"], keep_first=64,
                      s_heads=z["width"] // 32, s_vdim=64, s_state=128, d_heads=z["width"] // 64, d_dim=64,
                      experts=z["experts"], top=z["top"], expert_ff=z["expert_ff"], shared_ff=z["shared_ff"])
            rec = {"bulodra_config": {k: list(v) if isinstance(v, tuple) else v for k, v in z.items()}}
            for label, cfg in (("bulodra", bulodra_config(**z)),
                               ("leguvik (equal width, vocab, attention heads and window, experts; 7 layers)",
                                leguvik_config(**lz))):
                m = sb.random_model(cfg, seed=0, dtype="bfloat16", device=dev, std=0.02)
                rec[label] = bench.model_points(m, args.prompt, args.batch, args.steps, args.warmup)
                del m
                torch.cuda.empty_cache()
            for rows in (args.prompt, args.batch):
                rec["kernels_rows_%d" % rows] = bulodra_kernels(bench, z, rows, args.prompt)
            result["sizes"][name] = rec
    ops.check_status()
    result["clocks"] = clocks.summary()
    print(json.dumps(result))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0,
                    help="run fewer layers than the model has (both numbers go into config)")
    ap.add_argument("--prefill-reps", type=int, default=3)
    ap.add_argument("--no-extras", action="store_true",
                    help="leave out the points beyond the headline configuration (the session "
                         "entry point, the 1.5B and 32B sizes)")
    ap.add_argument("--layers-32b", type=int, default=0,
                    help="run the 32B sizes with fewer than their 64 layers (both numbers are recorded)")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one phase only and print a short line (small cases for profilers)")
    ap.add_argument("--eager", action="store_true",
                    help="with --only decode: launch the step kernel by kernel, not as a graph")
    ap.add_argument("--arch", choices=["qwen2", "zolulix", "mefupel", "leguvik", "bulodra"], default="qwen2",
                    help="zolulix: that design's prefill and decode throughput and its kernels alone, "
                         "beside the Qwen2.5 decoder of equal sizes (its own JSON line; the default "
                         "workload is unchanged); mefupel: the same for that design, beside Zolulix and "
                         "Qwen2.5 models of equal sizes; leguvik: the same for that design, beside Mefupel "
                         "models of equal sizes; bulodra: the same for that design, beside Leguvik models of "
                         "equal sizes")
    ap.add_argument("--sizes", default="", help="with --arch zolulix / mefupel / leguvik / bulodra: which of its sizes to run (comma separated)")
    ap.add_argument("--prompt", type=int, default=2048, help="with --arch zolulix / mefupel / leguvik / bulodra: prompt length")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        print("bench.py: this library runs on one GPU; --gpus N with N > 1 is not built")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.arch == "zolulix":
        return run_zolulix(args)
    if args.arch == "mefupel":
        return run_mefupel(args)
    if args.arch == "leguvik":
        return run_leguvik(args)
    if args.arch == "bulodra":
        return run_bulodra(args)
    return run(args)


if __name__ == "__main__":
    sys.exit(main())
