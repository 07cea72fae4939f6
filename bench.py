#!/usr/bin/env python3
"""Decode and prefill throughput of the GPT-2 engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--preset gpt2] [--batch 8]

A step is one decode step of the whole batch: every sequence goes on by one token.  The default run has
the layer sizes of the GPT-2 small configuration with random weights (seeded, synthetic token ids), a
batch of 8 and a context of 1,024: the sequences start from 512-token prompts and decode to 1,024 (16 warm-up
steps, then the 496 timed ones).
One JSON line is printed:

  value      decoded tokens a second, K steps timed on the device with CUDA events after W warm-up steps;
             the sampled tokens feed the next step on the device
  e2e        the same through the Python entry point (`Model.generate_ids`): every step copies its input
             tokens from pinned host memory to the device and reads the sampled tokens back
  prefill    one step of 2 x 1,024 prompt tokens: tokens a second, and its flops / time / the bf16 peak; the
             engine replays a captured graph for a step of a shape it has run before, which the timed
             repetitions are; `ms_new_shape` is the same step launched kernel by kernel from the host, as
             the first step of a new shape is
  roofline   decode: bytes the step has to read (every weight it uses once, the cache of the live
             sequences) / its time, against the HBM copy peak
  points     decode tokens a second at batch 1 and 64

Peaks come from MEASURED_PEAKS.json beside this file when the driver wrote it, else from the fallback
figures 6.65 TB/s and 1.59 PFLOP/s.  The working set of a step (weights + cache, > 400 MB) is larger than
the 126 MB L2, so no L2 flush is issued between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
PROMPT_LEN = 512


def peaks(root: str = ROOT):
    """(HBM copy GB/s, bf16 TFLOP/s of a burst, "measured" | "fallback").  The measured file gives `hbm_gbs` and
    `bf16_tflops` as numbers (a figure wrapped as {"value": x} is read too); anything else in it, or a file that
    does not parse, leaves the fallback figure for that peak."""
    path = os.path.join(root, "MEASURED_PEAKS.json")
    hbm, tf, src = FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"

    def number(v):
        if isinstance(v, dict):
            v = v.get("value")
        if isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0:
            return float(v)
        return None

    try:
        with open(path) as f:
            p = json.load(f)
    except (OSError, ValueError):
        return hbm, tf, src
    if isinstance(p, dict):
        got_hbm, got_tf = number(p.get("hbm_gbs")), number(p.get("bf16_tflops"))
        if got_hbm is not None:
            hbm, src = got_hbm, "measured"
        if got_tf is not None:
            tf, src = got_tf, "measured"
    return hbm, tf, src


class ClockSampler:
    """Samples SM clocks and throttle reasons while a timed region runs: through NVML every few
    milliseconds (read-only queries), or with nvidia-smi if the NVML module is missing."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, period_s: float = 0.005):
        self.samples, self.proc, self.thread = [], None, None
        self.period_s, self.stop = period_s, threading.Event()

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(0)
            pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
            self.thread = threading.Thread(target=self._poll, args=(pynvml, handle), daemon=True)
            self.thread.start()
            return self
        except Exception:  # noqa: BLE001 - no NVML: ask nvidia-smi instead
            pass
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _poll(self, pynvml, handle):
        reasons_of = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
        try:
            mx = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
            while not self.stop.is_set():
                sm = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
                bits = int(reasons_of(handle))
                flags = ["Active" if bits & self.REASON_BITS[n] else "Not Active"
                         for n in ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")]
                self.samples.append(", ".join([str(sm), str(mx)] + flags))
                self.stop.wait(self.period_s)
        except Exception:  # noqa: BLE001 - a failed query ends the sampling, not the benchmark
            pass

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def __exit__(self, *exc):
        self.stop.set()
        if self.proc is not None:
            self.proc.terminate()          # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        elif self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            parts = [p.strip() for p in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def step_bytes(model, engine, slots) -> int:
    """Bytes a decode step has to read: every weight it uses once (the position table only the rows of
    this step) and the keys and values of the live sequences."""
    cfg = model.config
    w = model.weight_bytes()
    wpe_all = cfg.n_positions * cfg.n_embd * (2 if model.act_dtype.itemsize == 2 else 4)
    wpe_used = len(slots) * cfg.n_embd * (2 if model.act_dtype.itemsize == 2 else 4)
    return w - wpe_all + wpe_used + engine.cache.live_kv_bytes(slots)


def prefill_flops(cfg, lens, n_logit_rows) -> float:
    d, f, L, H = cfg.n_embd, cfg.inner_dim, cfg.n_layer, cfg.n_head
    T = sum(lens)
    gemm = 2.0 * T * (3 * d * d + d * d + 2 * d * f) * L
    attn = sum(4.0 * (d // H) * (s * (s + 1) / 2) * H for s in lens) * L
    head = 2.0 * n_logit_rows * d * cfg.vocab_size
    return gemm + attn + head


def make_model_dir(preset: str, n_layer: int | None, tmp: str) -> str:
    import vlrf_b200.models  # noqa: F401
    from vlrf_b200.config import load_preset
    from vlrf_b200.weights import write_random_model
    cfg = load_preset(preset)
    if n_layer is not None:
        cfg["n_layer"] = n_layer
    return str(write_random_model(cfg, 1234, os.path.join(tmp, "model")))


def random_prompts(vocab, batch, length, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (batch, length), generator=g).tolist()


def decode_device(model_dir, batch, steps, warmup, dtype="bfloat16"):
    """K decode steps timed on the device; tokens stay on the device between steps."""
    import torch
    from vlrf_b200.csrc import ops
    from vlrf_b200.engine import Engine, StepEntry, load_model
    from vlrf_b200.engine.decode import DecodeSession
    model = load_model(model_dir, dtype)
    cfg = model.config
    ctx_len = cfg.n_positions
    steps = min(steps, ctx_len - PROMPT_LEN - warmup)
    engine = Engine(model, max_tokens=batch * ctx_len, n_slots=batch)
    prompts = random_prompts(cfg.vocab_size, batch, PROMPT_LEN, 1)
    slots = [engine.start_sequence() for _ in range(batch)]
    out = torch.zeros(batch, dtype=torch.int32, device=model.device)
    for b0 in range(0, batch, 8):      # prompts in steps of 8 sequences
        idx = list(range(b0, min(batch, b0 + 8)))
        logits = engine.step([StepEntry(slots[i], prompts[i], [PROMPT_LEN - 1]) for i in idx])
        ops.sample(logits, len(idx), out[b0:b0 + len(idx)])
    sess = DecodeSession(engine, slots, use_graph=True)
    sess.reserve_ahead(warmup + steps + 1)
    sess.set_tokens(out)
    for _ in range(warmup):
        sess.step_greedy(out)
    torch.cuda.synchronize()
    bytes_first = step_bytes(model, engine, slots)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler() as clk:
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            sess.step_greedy(out)        # model + argmax + hand-over to the next step: one replayed graph
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    bytes_last = step_bytes(model, engine, slots)
    engine.check_device_errors()
    launches = steps * sess.kernels_per_step              # the step's kernels, sampling included (replayed)
    return dict(tok_s=batch * steps / (ms / 1e3), ms_per_step=ms / steps, steps=steps,
                bytes_per_step=(bytes_first + bytes_last) / 2, clocks=clk.summary(), launches=launches,
                kernels_per_step=sess.kernels_per_step, mean_context=PROMPT_LEN + warmup + steps / 2,
                weight_bytes=model.weight_bytes(), n_layer=cfg.n_layer)


def decode_e2e(model_dir, batch, steps, warmup, dtype="bfloat16"):
    """The same K steps through Model.generate_ids: host tokens in and out at every step."""
    import torch
    from vlrf_b200 import Model, SamplingParams
    model = Model.load(model_dir, dtype=dtype, max_tokens=batch * 1024, n_slots=batch)
    cfg = model.config
    steps = min(steps, cfg.n_positions - PROMPT_LEN - warmup - 2)
    prompts = random_prompts(cfg.vocab_size, batch, PROMPT_LEN, 1)
    marks = {}
    count = [0]

    def on_token(index, tok):
        if index != 0:
            return True
        count[0] += 1                       # token number of request 0 = step number
        if count[0] == warmup + 1:          # prompt step and W decode steps are done
            torch.cuda.synchronize()
            marks["t0"] = time.perf_counter()
            marks["h2d0"], marks["d2h0"] = model.backend.h2d_bytes, model.backend.d2h_bytes
        elif count[0] == warmup + 1 + steps:
            torch.cuda.synchronize()
            marks["t1"] = time.perf_counter()
            marks["h2d1"], marks["d2h1"] = model.backend.h2d_bytes, model.backend.d2h_bytes
        return True

    params = SamplingParams(max_new_tokens=warmup + steps + 2, do_sample=False, stop_token_ids=())
    model.generate_ids(prompts, params, on_token=on_token)
    dt = marks["t1"] - marks["t0"]
    return dict(tok_s=batch * steps / dt, h2d=(marks["h2d1"] - marks["h2d0"]) / steps,
                d2h=(marks["d2h1"] - marks["d2h0"]) / steps, steps=steps)


def prefill_device(model_dir, dtype="bfloat16", reps=5, replay=True):
    """One step of 2 x 1,024 prompt tokens.  replay: the engine replays a captured graph for a step whose shape
    it has seen before (the default); without it every kernel is launched from the host, as for a new shape."""
    import torch
    from vlrf_b200.engine import Engine, StepEntry, load_model
    model = load_model(model_dir, dtype)
    cfg = model.config
    n_seq, length = 2, min(1024, cfg.n_positions)
    engine = Engine(model, max_tokens=n_seq * length, n_slots=n_seq)
    engine.capture_repeated_steps = replay
    import numpy as np
    # host token ids as int32 arrays (a Python list of a thousand ids costs about 30 us to convert, inside the step)
    prompts = [np.asarray(p, dtype=np.int32) for p in random_prompts(cfg.vocab_size, n_seq, length, 2)]
    times = []
    for r in range(reps + 2):
        slots = [engine.start_sequence() for _ in range(n_seq)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.step([StepEntry(s, p, [length - 1]) for s, p in zip(slots, prompts)])
        e1.record()
        torch.cuda.synchronize()
        if r >= 2:
            times.append(e0.elapsed_time(e1))
        for s in slots:
            engine.end_sequence(s)
    engine.check_device_errors()
    ms = statistics.median(times)
    return dict(tokens=n_seq * length, ms=ms, flops=prefill_flops(cfg, [length] * n_seq, n_seq))


# ---- a second design beside its closest existing model (--design) ---------------------------------------------------------

#: Kuvusun at two sizes that resemble a real model's layers, each beside a GPT-2 of the same width, depth, heads and
#: dense inner size.  Layers: queries through a latent + dense feed-forward; rotated part + routed experts; the same
#: reading the cache of the layer before; queries through a latent + routed experts.
DESIGN_SIZES = {
    "s": dict(width=1024, heads=16, dim=64, rot=32, vdim=64, kv_rank=256, q_rank=384, ff=4096, experts=16, top=2,
              expert_ff=1024, shared_ff=1024, vocab=32000),
    "m": dict(width=2048, heads=16, dim=128, rot=64, vdim=128, kv_rank=512, q_rank=768, ff=8192, experts=32, top=4,
              expert_ff=1408, shared_ff=2816, vocab=32000),
}


def kuvusun_config(z: dict) -> dict:
    att1 = {"type": "latent_attention", "mixer": {"heads": z["heads"], "dim": z["dim"], "vdim": z["vdim"], "kv_rank": z["kv_rank"],
                                                  "q_rank": z["q_rank"], "scale": z["dim"] ** -0.5}}

    def att2(kv_from=None):
        m = {"heads": z["heads"], "dim": z["dim"], "vdim": z["vdim"], "kv_rank": z["kv_rank"], "rot_dim": z["rot"],
             "rot": {"base": 10000.0, "dims": z["rot"]}, "scale": (z["dim"] + z["rot"]) ** -0.5}
        if kv_from is not None:
            m["kv_from"] = kv_from
        return {"type": "latent_attention_2", "mixer": m}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"]},
           "shared": {"ff": z["shared_ff"]}}
    layers = [dict(att1, mlp={"kind": "dense", "ff": z["ff"]}), dict(att2(), mlp=moe), dict(att2(1), mlp=moe), dict(att1, mlp=moe)]
    return {"architecture": "Kuvusun", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5, "groups": 4}, "layers": layers}


#: Kotisun at two sizes that resemble a real model's layers, each beside a GPT-2 of the same width, depth and heads whose
#: (ungated) feed-forward has about the parameters of the gated one.  Four layers, the middle two run twice.
KOTISUN_SIZES = {
    "s": dict(width=1024, heads=16, kv_heads=4, dim=64, vdim=96, window=512, rot=32, r_heads=32, r_vdim=64, state=64, groups=4,
              norm_groups=4, ff_gated=2816, ff=4096, streams=4, vocab=32000),
    "m": dict(width=2048, heads=16, kv_heads=2, dim=128, vdim=128, window=1024, rot=64, r_heads=32, r_vdim=128, state=128, groups=8,
              norm_groups=8, ff_gated=5632, ff=8192, streams=4, vocab=32000),
}


def kotisun_config(z: dict) -> dict:
    left = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
            "mask": {"size": z["window"]}, "rot": {"base": 10000.0, "dims": z["rot"], "scaling": {"factor": 2.0}}}
    right = {"heads": z["r_heads"], "vdim": z["r_vdim"], "state": z["state"], "groups": z["groups"], "conv": 4, "norm_groups": z["norm_groups"]}
    layer = {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 0.7, "right_scale": 0.7},
             "mlp": {"kind": "dense", "ff": z["ff_gated"]}}
    return {"architecture": "Kotisun", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "streams": z["streams"], "loop": {"start": 1, "stop": 2, "times": 2}, "logit_softcap": 30.0, "layers": [layer] * 3}


def gpt2_config_like(z: dict) -> dict:
    return dict(model_type="gpt2", n_layer=4, n_embd=z["width"], n_head=z["heads"], n_inner=z["ff"], vocab_size=z["vocab"],
                n_positions=2048, layer_norm_epsilon=1e-5, activation_function="gelu_new", tie_word_embeddings=True,
                bos_token_id=0, eos_token_id=0)


def design_point(model_dir: str, prompt_len: int, batches, steps: int, warmup: int) -> dict:
    """Prefill (2 sequences of prompt_len tokens, replayed graph, median of 5) and decode (per batch size: `steps`
    replayed steps from contexts of prompt_len) of one model, and the device time of every kernel entry point in one
    prompt step and one decode step launched kernel by kernel."""
    import numpy as np
    import torch
    from vlrf_b200 import log
    from vlrf_b200.csrc import ops
    from vlrf_b200.engine import Engine, StepEntry, load_model
    from vlrf_b200.engine.decode import DecodeSession
    model = load_model(model_dir, "bfloat16")
    vocab = model.vocab_size
    out = {"weights_mib": round(model.weight_bytes() / 2**20, 1)}
    # prefill
    engine = Engine(model, max_tokens=2 * prompt_len, n_slots=2)
    prompts = [np.asarray(p, dtype=np.int32) for p in random_prompts(vocab, 2, prompt_len, 2)]
    times = []
    for r in range(8):
        if r == 7:                      # the last repetition: kernel by kernel, each timed
            engine.capture_repeated_steps = False
            log.timers.reset(); log.timers.enable(True)
        slots = [engine.start_sequence() for _ in range(2)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.step([StepEntry(s, p, [prompt_len - 1]) for s, p in zip(slots, prompts)])
        e1.record()
        torch.cuda.synchronize()
        if 2 <= r < 7:
            times.append(e0.elapsed_time(e1))
        for s in slots:
            engine.end_sequence(s)
    log.timers.enable(False)
    engine.check_device_errors()
    out["prefill"] = {"tokens": 2 * prompt_len, "ms": round(statistics.median(times), 4),
                      "tok_s": round(2 * prompt_len / (statistics.median(times) / 1e3), 1),
                      "kernels_us": {k: [n, round(1e3 * ms, 1)] for k, n, ms, _ in log.timers.report()}}
    del engine
    # decode
    out["decode"] = {}
    for batch in batches:
        engine = Engine(model, max_tokens=batch * (prompt_len + 64 * (2 + (warmup + steps) // 64)), n_slots=batch)
        prompts = random_prompts(vocab, batch, prompt_len, 1)
        slots = [engine.start_sequence() for _ in range(batch)]
        tok = torch.zeros(batch, dtype=torch.int32, device=model.device)
        for b0 in range(0, batch, 8):
            idx = list(range(b0, min(batch, b0 + 8)))
            logits = engine.step([StepEntry(slots[i], prompts[i], [prompt_len - 1]) for i in idx])
            ops.sample(logits, len(idx), tok[b0:b0 + len(idx)])
        sess = DecodeSession(engine, slots, use_graph=True)
        sess.reserve_ahead(warmup + steps + 2)
        sess.set_tokens(tok)
        for _ in range(warmup):
            sess.step_greedy(tok)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            sess.step_greedy(tok)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        # one more step kernel by kernel, each timed
        plain = DecodeSession(engine, slots, use_graph=False)
        plain.set_tokens(tok)
        plain.step_greedy(tok)
        log.timers.reset(); log.timers.enable(True)
        plain.step_greedy(tok)
        log.timers.enable(False)
        engine.check_device_errors()
        out["decode"][f"b{batch}"] = {"ms_per_step": round(ms, 4), "tok_s": round(batch / (ms / 1e3), 1),
                                      "kernels_per_step": sess.kernels_per_step, "cache_mib": round(engine.cache.live_kv_bytes(slots) / 2**20, 1),
                                      "kernels_us": {k: [n, round(1e3 * t, 1)] for k, n, t, _ in log.timers.report()}}
        del sess, plain, engine
    return out


def design_kernels(z: dict, hbm_gbs: float, bf16_tflops: float) -> dict:
    """The design's own kernels alone, each beside the like kernel of GPT-2 at equal size: 20 launches back to back
    between two events after 3 warm-up launches, inputs rotated over buffers that together exceed L2 where a kernel is
    bound by bytes.  Fractions are of the measured copy bandwidth or bf16 product throughput."""
    import types
    import torch
    from vlrf_b200.csrc import ops
    from vlrf_b200.parts.context import Workspace
    dev, bf = "cuda", torch.bfloat16
    H, C, R, dim, vdim, width = z["heads"], z["kv_rank"], z["rot"], z["dim"], z["vdim"], z["width"]
    D = C + R
    dev_err = torch.zeros(1, dtype=torch.int32, device=dev)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)

    def timed(fn, reps=20):
        for i in range(3):
            fn(i)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for i in range(reps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3           # microseconds a launch

    out = {}
    # -- decode attention: 64 sequences at context 1,024 ----------------------------------------------------------------
    B, ctxlen = 64, 1024
    nblk = B * ctxlen // 64
    table = torch.arange(nblk, dtype=torch.int32, device=dev).view(B, ctxlen // 64).contiguous()
    slots, pos = i32(list(range(B))), i32([ctxlen - 1] * B)
    n_buf = max(2, int(300e6 // (nblk * 64 * D * 2)) + 1)
    caches = [torch.randn(nblk, 64, D, device=dev).to(bf) for _ in range(n_buf)]
    qp = torch.randn(B, H * D, device=dev).to(bf)
    o = torch.zeros(B, H * C, dtype=bf, device=dev)
    ctx = types.SimpleNamespace(max_new=1, n_seqs=B, seq_slot=slots, seq_start=i32(list(range(B + 1))), seq_pos0=pos,
                                max_context=ctxlen, ws=Workspace(dev))
    us = timed(lambda i: ops.attention_latent(qp, caches[i % n_buf], C, R, table, slots, pos, o, B, H, 0.1, 0, dev_err, ctx=ctx))
    nbytes = B * ctxlen * D * 2
    out["attention_decode"] = {"kuvusun": {"us": round(us, 1), "gb_s": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / hbm_gbs, 3),
                                           "mib": round(nbytes / 2**20, 1)}}
    del caches
    dh = width // H
    n_buf = max(2, int(300e6 // (2 * nblk * H * 64 * dh * 2)) + 1)
    ks = [torch.randn(nblk, H, 64, dh, device=dev).to(bf) for _ in range(n_buf)]
    vs = [torch.randn(nblk, H, 64, dh, device=dev).to(bf) for _ in range(n_buf)]
    qkv = torch.randn(B, 3 * width, device=dev).to(bf)
    o2 = torch.zeros(B, width, dtype=bf, device=dev)
    n_split = ops.decode_splits(B, H, ctxlen)
    ws = Workspace(dev)
    partials = counters = None
    if n_split > 1 and ops.attention_decode_needs_scratch(dh, n_split):
        partials = ws.get("p", B * H * n_split, dh + 2, torch.float32)
        counters = ws.get_zeroed("c", B * H, torch.int32)
    us = timed(lambda i: ops.attention_decode(qkv, 0, ks[i % n_buf], vs[i % n_buf], table, slots, pos, o2, B, H, H, dh, 0.1, 0, n_split,
                                              partials, counters, dev_err))
    nbytes = 2 * B * ctxlen * H * dh * 2
    out["attention_decode"]["gpt2"] = {"us": round(us, 1), "gb_s": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / hbm_gbs, 3),
                                       "mib": round(nbytes / 2**20, 1)}
    # -- prompt attention: 2 sequences of 1,024 tokens -----------------------------------------------------------------
    S, L = 2, 1024
    T = S * L
    tok_slot = i32([s for s in range(S) for _ in range(L)])
    tok_pos = i32(list(range(L)) * S)
    pctx = types.SimpleNamespace(max_new=L, n_seqs=S, seq_slot=i32(list(range(S))), seq_start=i32([0, L, 2 * L]), seq_pos0=i32([0, 0]),
                                 max_context=L, ws=Workspace(dev))
    ptable = torch.arange(S * L // 64, dtype=torch.int32, device=dev).view(S, L // 64).contiguous()
    cache = torch.randn(S * L // 64, 64, D, device=dev).to(bf)
    qpp = torch.randn(T, H * D, device=dev).to(bf)
    op = torch.zeros(T, H * C, dtype=bf, device=dev)
    us = timed(lambda i: ops.attention_latent(qpp, cache, C, R, ptable, tok_slot, tok_pos, op, T, H, 0.1, 0, dev_err, ctx=pctx), reps=10)
    pairs = S * L * (L + 1) / 2
    done = 2.0 * pairs * H * (D + C)                           # what the kernel multiplies (queries carried into latent space)
    asked = 2.0 * pairs * H * (dim + R + vdim)                 # what the design's equations ask for, keys and values per head
    out["attention_prompt"] = {"kuvusun": {"us": round(us, 1), "tflops_done": round(done / us / 1e6, 1), "frac_done": round(done / us / 1e6 / bf16_tflops, 3),
                                           "tflops_asked": round(asked / us / 1e6, 1), "frac_asked": round(asked / us / 1e6 / bf16_tflops, 4)}}
    # the same step when its sequences begin at position 0: keys and values formed, attention over plain rows
    if ops.attention_rows_takes(bf, dim, R, vdim, H):
        qn_, qr_ = torch.randn(T, H * dim, device=dev).to(bf), torch.randn(T, H * R, device=dev).to(bf)
        kn_, kr_, vv_ = torch.randn(T, H * dim, device=dev).to(bf), torch.randn(T, R, device=dev).to(bf), torch.randn(T, H * vdim, device=dev).to(bf)
        om = torch.zeros(T, H * vdim, dtype=bf, device=dev)
        us = timed(lambda i: ops.attention_rows(qn_, qr_, kn_, kr_, vv_, pctx.seq_start, om, S, L, H, dim, R, vdim, 0.1), reps=10)
        out["attention_prompt"]["kuvusun_rows"] = {"us": round(us, 1), "tflops": round(asked / us / 1e6, 1), "frac": round(asked / us / 1e6 / bf16_tflops, 3)}
    k1, v1 = ks[0][:S * L // 64], vs[0][:S * L // 64]
    qkvp = torch.randn(T, 3 * width, device=dev).to(bf)
    op2 = torch.zeros(T, width, dtype=bf, device=dev)
    if ops.attention_prefill_takes(bf, dh, 64, 3 * width, 0):
        n_parts = ops.attention_prefill_parts(bf, S, L, H, dh, 64, 3 * width, 0)
        pp = cc = None
        if n_parts > 1:
            nf, nc = ops.attention_prefill_scratch(S, L, H, n_parts)
            pp, cc = ws.get("pp", nf, 1, torch.float32), ws.get_zeroed("pc", nc, torch.int32)
        us = timed(lambda i: ops.attention_prefill(qkvp, 0, k1, v1, ptable, pctx.seq_slot, pctx.seq_start, pctx.seq_pos0, op2, T, S, L, H, H,
                                                   dh, 0.1, 0, dev_err, n_parts, pp, cc), reps=10)
        fl = 4.0 * pairs * H * dh
        out["attention_prompt"]["gpt2"] = {"us": round(us, 1), "tflops_done": round(fl / us / 1e6, 1), "frac_done": round(fl / us / 1e6 / bf16_tflops, 3)}
    del ks, vs
    # -- the experts' first product: prompt step (T · top rows) and decode step (64 · top rows), rows dealt evenly -------
    E, top, ff = z["experts"], z["top"], z["expert_ff"]
    w = (torch.randn(E, 2 * ff, width, device=dev) * 0.02).to(bf)
    for label, rows in (("experts_prompt", T * top), ("experts_decode", 64 * top)):
        x = torch.randn(rows, width, device=dev).to(bf)
        y = torch.zeros(rows, 2 * ff, dtype=bf, device=dev)
        offs = i32([rows * e // E for e in range(E + 1)])
        us = timed(lambda i: ops.linear_grouped(x, w, y, offs, rows))
        fl, nbytes = 2.0 * rows * 2 * ff * width, E * 2 * ff * width * 2
        out[label] = {"kuvusun": {"us": round(us, 1), "tflops": round(fl / us / 1e6, 1), "frac_tensor": round(fl / us / 1e6 / bf16_tflops, 3),
                                  "gb_s": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / hbm_gbs, 3)}}
    n_w = max(2, int(300e6 // (z["ff"] * width * 2)) + 1)
    wd = [(torch.randn(z["ff"], width, device=dev) * 0.02).to(bf) for _ in range(n_w)]
    for label, rows in (("experts_prompt", T), ("experts_decode", 64)):
        x = torch.randn(rows, width, device=dev).to(bf)
        y = torch.zeros(rows, z["ff"], dtype=bf, device=dev)
        us = timed(lambda i: ops.linear(x, wd[i % n_w], None, y))
        fl, nbytes = 2.0 * rows * z["ff"] * width, z["ff"] * width * 2
        out[label]["gpt2"] = {"us": round(us, 1), "tflops": round(fl / us / 1e6, 1), "frac_tensor": round(fl / us / 1e6 / bf16_tflops, 3),
                              "gb_s": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / hbm_gbs, 3)}
    # -- the products per head around the attention (queries into latent space), prompt step --------------------------------
    qn = torch.randn(T, H, dim, device=dev).to(bf)
    wk = (torch.randn(H, C, dim, device=dev) * 0.05).to(bf)
    us = timed(lambda i: ops.linear_heads(qn, wk, qpp.view(T, H, D)[:, :, :C], T))
    fl = 2.0 * T * H * C * dim
    out["heads_prompt"] = {"kuvusun": {"us": round(us, 1), "tflops": round(fl / us / 1e6, 1), "frac_tensor": round(fl / us / 1e6 / bf16_tflops, 3)}}
    return out


def kotisun_kernels(z: dict, hbm_gbs: float, bf16_tflops: float) -> dict:
    """Kotisun's own kernels alone, each beside the like kernel of GPT-2 at equal width where there is one (timed as in
    `design_kernels`): windowed attention in a decode step and in a prompt step, the recurrence in both, the
    convolution, and the reads and writes of the residual's streams beside GPT-2's LayerNorm."""
    import types
    import torch
    from vlrf_b200.csrc import ops
    from vlrf_b200.parts.context import Workspace
    dev, bf = "cuda", torch.bfloat16
    H, G, dk, dv, W, width = z["heads"], z["kv_heads"], z["dim"], z["vdim"], z["window"], z["width"]
    dev_err = torch.zeros(1, dtype=torch.int32, device=dev)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)   # noqa: E731

    def timed(fn, reps=20):
        for i in range(3):
            fn(i)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for i in range(reps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3           # microseconds a launch

    def bytes_point(us, nbytes):
        return {"us": round(us, 1), "gb_s": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / hbm_gbs, 3), "mib": round(nbytes / 2**20, 1)}

    def flops_point(us, fl):
        return {"us": round(us, 1), "tflops": round(fl / us / 1e6, 1), "frac_tensor": round(fl / us / 1e6 / bf16_tflops, 4)}

    # (a fifth of a second of work first: the first kernel measured in a process otherwise runs before the GPU has left its
    # idle clocks, which the three warm-up launches of a 20 us kernel do not outlast)
    warm_x, warm_y = torch.zeros(4096, 4 * 1024, device=dev), torch.zeros(4096, 1024, device=dev)
    warm_m, warm_b = torch.eye(4, device=dev), torch.zeros(4, device=dev)
    t_end = time.time() + 0.2
    while time.time() < t_end:
        ops.streams_write(warm_x, 4, warm_m, warm_b, warm_y, 4096)
        torch.cuda.synchronize()
    del warm_x, warm_y
    out = {}
    # -- decode attention: 64 sequences at context 1,024 (of which the window is read) --------------------------------------
    B, ctxlen = 64, 1024
    nblk = B * ctxlen // 64
    # (blocks dealt at random, as a cache that has served other sequences before hands them out)
    table = torch.randperm(nblk, generator=torch.Generator().manual_seed(5)).to(dtype=torch.int32, device=dev).view(B, ctxlen // 64).contiguous()
    slots, pos = i32(list(range(B))), i32([ctxlen - 1] * B)
    seen = min(W, ctxlen)
    n_buf = max(2, int(300e6 // (B * seen * G * (dk + dv) * 2)) + 1)
    ks = [torch.randn(nblk, G, 64, dk, device=dev).to(bf) for _ in range(n_buf)]
    vs = [torch.randn(nblk, G, 64, dv, device=dev).to(bf) for _ in range(n_buf)]
    q = torch.randn(B, H * dk, device=dev).to(bf)
    o = torch.zeros(B, H * dv, dtype=bf, device=dev)
    ctx = types.SimpleNamespace(n_tokens=B, max_new=1, n_seqs=B, seq_slot=slots, seq_start=i32(list(range(B + 1))), seq_pos0=pos, tok_slot=slots,
                                tok_pos=pos, max_context=ctxlen, ws=Workspace(dev), dev_err=dev_err)
    us = timed(lambda i: ops.attention_window_step(q, ks[i % n_buf], vs[i % n_buf], table, o, ctx, H, G, dk, dv, 0.1, W, 1.0))
    out["attention_decode"] = {"kotisun": bytes_point(us, B * seen * G * (dk + dv) * 2)}
    del ks, vs
    dh = width // H
    n_buf = max(2, int(300e6 // (2 * nblk * H * 64 * dh * 2)) + 1)
    ks = [torch.randn(nblk, H, 64, dh, device=dev).to(bf) for _ in range(n_buf)]
    vs = [torch.randn(nblk, H, 64, dh, device=dev).to(bf) for _ in range(n_buf)]
    qkv = torch.randn(B, 3 * width, device=dev).to(bf)
    o2 = torch.zeros(B, width, dtype=bf, device=dev)
    n_split = ops.decode_splits(B, H, ctxlen)
    ws = Workspace(dev)
    partials = counters = None
    if n_split > 1 and ops.attention_decode_needs_scratch(dh, n_split):
        partials = ws.get("p", B * H * n_split, dh + 2, torch.float32)
        counters = ws.get_zeroed("c", B * H, torch.int32)
    us = timed(lambda i: ops.attention_decode(qkv, 0, ks[i % n_buf], vs[i % n_buf], table, slots, pos, o2, B, H, H, dh, 0.1, 0, n_split,
                                              partials, counters, dev_err))
    out["attention_decode"]["gpt2"] = bytes_point(us, 2 * B * ctxlen * H * dh * 2)
    # -- prompt attention: 2 sequences of 1,024 tokens --------------------------------------------------------------------
    S, L = 2, 1024
    T = S * L
    pctx = types.SimpleNamespace(n_tokens=T, max_new=L, n_seqs=S, seq_slot=i32(list(range(S))), seq_start=i32([0, L, 2 * L]), seq_pos0=i32([0, 0]),
                                 tok_slot=i32([s for s in range(S) for _ in range(L)]), tok_pos=i32(list(range(L)) * S), max_context=L,
                                 ws=Workspace(dev), dev_err=dev_err)
    ptable = torch.arange(S * L // 64, dtype=torch.int32, device=dev).view(S, L // 64).contiguous()
    kp, vp = torch.randn(S * L // 64, G, 64, dk, device=dev).to(bf), torch.randn(S * L // 64, G, 64, dv, device=dev).to(bf)
    qp = torch.randn(T, H * dk, device=dev).to(bf)
    op = torch.zeros(T, H * dv, dtype=bf, device=dev)
    us = timed(lambda i: ops.attention_window_step(qp, kp, vp, ptable, op, pctx, H, G, dk, dv, 0.1, W, 1.0), reps=10)
    pairs = S * sum(min(i + 1, W) for i in range(L))
    out["attention_prompt"] = {"kotisun": flops_point(us, 2.0 * pairs * H * (dk + dv))}
    k1, v1 = ks[0][:S * L // 64], vs[0][:S * L // 64]
    qkvp = torch.randn(T, 3 * width, device=dev).to(bf)
    op2 = torch.zeros(T, width, dtype=bf, device=dev)
    if ops.attention_prefill_takes(bf, dh, 64, 3 * width, 0):
        n_parts = ops.attention_prefill_parts(bf, S, L, H, dh, 64, 3 * width, 0)
        pp = cc = None
        if n_parts > 1:
            nf, nc = ops.attention_prefill_scratch(S, L, H, n_parts)
            pp, cc = ws.get("pp", nf, 1, torch.float32), ws.get_zeroed("pc", nc, torch.int32)
        us = timed(lambda i: ops.attention_prefill(qkvp, 0, k1, v1, ptable, pctx.seq_slot, pctx.seq_start, pctx.seq_pos0, op2, T, S, L, H, H,
                                                   dh, 0.1, 0, dev_err, n_parts, pp, cc), reps=10)
        out["attention_prompt"]["gpt2"] = flops_point(us, 4.0 * (S * L * (L + 1) / 2) * H * dh)
    del ks, vs
    # -- the recurrence: prompt step (2 × 1,024 tokens) and decode step (64 sequences); bytes: the state read and written, and the rows
    Hs, P, N, Gs, taps = z["r_heads"], z["r_vdim"], z["state"], z["groups"], 4
    inner, channels = Hs * P, Hs * P + 2 * Gs * N
    ld = 2 * inner + 2 * Gs * N + Hs
    state_row = Hs * N * P + (taps - 1) * channels
    conv_w, conv_b = torch.randn(channels, taps, device=dev) * 0.3, torch.zeros(channels, device=dev)
    dt_bias, a_log, dsk = torch.full((Hs,), -1.0, device=dev), torch.zeros(Hs, device=dev), torch.ones(Hs, device=dev)
    norm_w = torch.ones(inner, device=dev)
    for label, c, rows, n_seq, new in (("prompt", pctx, T, S, L), ("decode", ctx, B, B, 1)):
        n_state = max(2, int(300e6 // (n_seq * 2 * state_row * 4)) + 1) if label == "decode" else 1
        states = [torch.zeros(n_seq, 2, state_row, device=dev) for _ in range(n_state)]
        proj = torch.randn(rows, ld, device=dev) * 0.5
        xbc, y = torch.zeros(rows, channels, device=dev), torch.zeros(rows, inner, device=dev)
        merged = torch.zeros(rows, inner, dtype=bf, device=dev)
        us = timed(lambda i: ops.ssd_conv(proj, inner, conv_w, conv_b, states[i % n_state], Hs * N * P, c.seq_slot, c.seq_start, c.seq_pos0, xbc,
                                          n_seq, new), reps=10)
        out["conv_" + label] = {"kotisun": bytes_point(us, rows * channels * 8)}
        us = timed(lambda i: ops.ssd_scan_step(xbc, proj, inner + channels, dt_bias, a_log, dsk, states[i % n_state], c, y, Hs, Gs, N, P), reps=10)
        nbytes = n_seq * 2 * Hs * N * P * 4 + rows * (channels + inner) * 4
        fl = 2.0 * rows * Hs * N * P * 2
        out["scan_" + label] = {"kotisun": dict(bytes_point(us, nbytes), tflops=round(fl / us / 1e6, 2))}
        us = timed(lambda i: ops.ssd_gate_norm(y, proj, 0, norm_w, z["norm_groups"], 1e-5, 1.0, merged, rows), reps=10)
        out["gate_norm_" + label] = {"kotisun": bytes_point(us, rows * inner * 10)}
        del states
    # -- the residual's streams beside GPT-2's LayerNorm: read + norm, and the write --------------------------------------------
    St = z["streams"]
    for label, rows in (("prompt", T), ("decode", B)):
        n_x = max(2, int(300e6 // (rows * St * width * 4)) + 1)
        xs = [torch.randn(rows, St * width, device=dev) for _ in range(n_x)]
        a, w_, mix, b = torch.ones(St, device=dev), torch.ones(width, device=dev), torch.eye(St, device=dev), torch.ones(St, device=dev)
        h, yv = torch.zeros(rows, width, dtype=bf, device=dev), torch.randn(rows, width, device=dev)
        us = timed(lambda i: ops.streams_read_norm(xs[i % n_x], St, a, w_, 1e-5, h))
        out["streams_read_" + label] = {"kotisun": bytes_point(us, rows * width * (4 * St + 2))}
        us = timed(lambda i: ops.streams_write(xs[i % n_x], St, mix, b, yv, rows))
        out["streams_write_" + label] = {"kotisun": bytes_point(us, rows * width * (8 * St + 4))}
        x1 = [torch.randn(rows, width, device=dev) for _ in range(n_x)]
        us = timed(lambda i: ops.layernorm(x1[i % n_x], w_, w_, 1e-5, h))
        out["streams_read_" + label]["gpt2"] = bytes_point(us, rows * width * 6)
        del xs, x1
    return out


#: Rakelorn at two sizes that resemble a real model's layers, beside a Kuvusun of the same width, heads, latent sizes and
#: experts (its closest relative in the framework: latent attention and routed experts) with as many layers as Rakelorn
#: has layer runs.  Rakelorn: attention, recurrence, attention, attention, the recurrence's layer running twice; every
#: layer with routed experts, of which the last `identity` router outputs return their input.
RAKELORN_SIZES = {
    "s": dict(DESIGN_SIZES["s"], gru=1024, identity=2, groups=3, keep=2),
    "m": dict(DESIGN_SIZES["m"], gru=2048, identity=4, groups=4, keep=2),
}


def rakelorn_config(z: dict) -> dict:
    att = {"type": "latent_attention", "mixer": {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot"], "vdim": z["vdim"],
                                                 "kv_rank": z["kv_rank"], "q_rank": z["q_rank"], "scale": (z["dim"] + z["rot"]) ** -0.5,
                                                 "rot": {"base": 10000.0, "dims": z["rot"]}}}
    gru = {"type": "mingru", "mixer": {"width": z["gru"]}}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]},
           "router": {"experts": z["experts"], "identity": z["identity"], "top": z["top"], "scale": 2.0,
                      "groups": {"count": z["groups"], "keep": z["keep"]}}}
    return {"architecture": "Rakelorn", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "loop": {"start": 1, "stop": 2, "times": 2}, "layers": [dict(att, mlp=moe), dict(gru, mlp=moe), dict(att, mlp=moe), dict(att, mlp=moe)]}


def kuvusun_config_like(z: dict) -> dict:
    """A Kuvusun of five layers (Rakelorn's layer runs), each with a rotated part, a gate and routed experts without a shared one."""
    m = {"heads": z["heads"], "dim": z["dim"], "vdim": z["vdim"], "kv_rank": z["kv_rank"], "rot_dim": z["rot"],
         "rot": {"base": 10000.0, "dims": z["rot"]}, "scale": (z["dim"] + z["rot"]) ** -0.5}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"]}}
    return {"architecture": "Kuvusun", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5, "groups": 4},
            "layers": [{"type": "latent_attention_2", "mixer": m, "mlp": moe}] * 5}


def rakelorn_kernels(z: dict, hbm_gbs: float, bf16_tflops: float) -> dict:
    """Rakelorn's own kernels alone, each beside the like kernel of Kuvusun at equal size (20 launches replayed as one graph, inputs rotated over more than L2): the
    norm with its token shift beside the norm in groups, the gated recurrence beside the element-wise gate, the router by
    scores beside the router by logits, the weighted sum with identity experts beside the one without, the gate per head
    beside the gate per column, and an expert's first product without a gate beside the gated one.  Attention, the
    products per head and the grouped products are the kernels that Kuvusun runs (`--design kuvusun` measures them)."""
    import types
    import torch
    from vlrf_b200.csrc import ops
    dev, bf = "cuda", torch.bfloat16
    width, W, H, vdim = z["width"], z["gru"], z["heads"], z["vdim"]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)   # noqa: E731

    def timed(fn, reps=20):
        """Microseconds a launch: the `reps` launches are captured as one graph (as a step's kernels are when the engine
        replays it), so that the host's time to issue a launch is no part of the number."""
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(reps):
                fn(i)
        graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3

    def bytes_point(us, nbytes):
        return {"us": round(us, 1), "gb_s": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / hbm_gbs, 3), "mib": round(nbytes / 2**20, 1)}

    # (a fifth of a second of work first, so that the first kernel measured does not run at idle clocks)
    warm = torch.zeros(4096, 4096, device=dev)
    t_end = time.time() + 0.2
    while time.time() < t_end:
        warm.add_(1.0)
        torch.cuda.synchronize()
    del warm
    out = {}
    S, L, B = 2, 1024, 64
    T = S * L
    pctx = types.SimpleNamespace(n_tokens=T, max_new=L, n_seqs=S, seq_slot=i32(list(range(S))), seq_start=i32([0, L, 2 * L]), seq_pos0=i32([0, 0]),
                                 tok_slot=i32([s for s in range(S) for _ in range(L)]), tok_pos=i32(list(range(L)) * S))
    dctx = types.SimpleNamespace(n_tokens=B, max_new=1, n_seqs=B, seq_slot=i32(list(range(B))), seq_start=i32(list(range(B + 1))),
                                 seq_pos0=i32([L] * B), tok_slot=i32(list(range(B))), tok_pos=i32([L] * B))
    ones_w, mu = torch.ones(width, device=dev), torch.full((width,), 0.5, device=dev)
    for label, c, rows in (("prompt", pctx, T), ("decode", dctx, B)):
        # -- the first norm: RMS norm + token shift, beside Kuvusun's norm in groups (which adds to the residual) ---------------
        n_x = max(2, int(300e6 // (rows * width * 4)) + 1)
        xs = [torch.randn(rows, width, device=dev) for _ in range(n_x)]
        state = torch.zeros(max(S, B), 2, width, device=dev)
        h = torch.zeros(rows, width, dtype=bf, device=dev)
        us = timed(lambda i: ops.rmsnorm_shift(xs[i % n_x], ones_w, mu, 1e-6, state, c, h))
        out["norm_" + label] = {"rakelorn": bytes_point(us, rows * width * 6)}
        acc = torch.zeros(rows, width, device=dev)
        us = timed(lambda i: ops.group_rmsnorm(xs[i % n_x], ones_w, 1e-5, 4, acc, accumulate=True, also=h))
        out["norm_" + label]["kuvusun"] = bytes_point(us, rows * width * 14)
        del xs
        # -- the recurrence beside an element-wise gate over as many rows (Kuvusun's like kernel: nothing of it recurs) --------
        n_p = max(2, int(300e6 // (rows * 3 * W * 4)) + 1)
        projs = [torch.randn(rows, 3 * W, device=dev) for _ in range(n_p)]
        st = torch.zeros(max(S, B), 2, W, device=dev)
        g = torch.zeros(rows, W, dtype=bf, device=dev)
        us = timed(lambda i: ops.mingru_scan(projs[i % n_p], 0, W, 2 * W, W, st, c, g))
        out["recurrence_" + label] = {"rakelorn": bytes_point(us, rows * W * 14)}
        us = timed(lambda i: ops.gate_mul(projs[i % n_p][:, :W], projs[i % n_p][:, W:2 * W], g, "silu", rows, W))
        out["recurrence_" + label]["kuvusun_gate"] = bytes_point(us, rows * W * 10)
        del projs
        # -- the router and the weighted sum ------------------------------------------------------------------------------
        E, n_id, top = z["experts"], z["identity"], z["top"]
        zl = torch.randn(rows, E + n_id, device=dev)
        ids = torch.zeros(rows, top, dtype=torch.int32, device=dev)
        rank, row_of = torch.zeros_like(ids), torch.zeros_like(ids)
        wts = torch.zeros(rows, top, device=dev)
        counts = torch.zeros(E, dtype=torch.int32, device=dev)
        corr = torch.zeros(E + n_id, device=dev)
        us = timed(lambda i: (counts.zero_(), ops.moe_route_scored(zl, E + n_id, top, z["groups"], z["keep"], n_id, 2.0, corr, None, ids, wts, rank, counts, rows)))
        us0 = timed(lambda i: counts.zero_())
        out["router_" + label] = {"rakelorn": {"us": round(us - us0, 1)}}
        us = timed(lambda i: (counts.zero_(), ops.moe_route(zl, E, top, False, None, ids, wts, rank, None, counts, rows)))
        out["router_" + label]["kuvusun"] = {"us": round(us - us0, 1)}
        counts.zero_()
        ops.moe_route_scored(zl, E + n_id, top, z["groups"], z["keep"], n_id, 2.0, corr, None, ids, wts, rank, counts, rows)
        offsets = torch.zeros(E + 1, dtype=torch.int32, device=dev)
        ops.moe_plan(counts, offsets, E)
        hin = torch.randn(rows, width, device=dev).to(bf)
        sorted_rows = torch.zeros(rows * top, width, dtype=bf, device=dev)
        ops.moe_gather(hin, ids, rank, offsets, sorted_rows, row_of, rows, top)
        n_e = max(2, int(300e6 // (rows * top * width * 4)) + 1)
        eos = [torch.randn(rows * top, width, device=dev) for _ in range(n_e)]
        y = torch.zeros(rows, width, device=dev)
        us = timed(lambda i: ops.moe_combine(eos[i % n_e], row_of, wts, top, None, None, y, rows, residual=y, ids=ids, h=hin))
        out["combine_" + label] = {"rakelorn": bytes_point(us, rows * width * (4 * top + 8 + 2))}
        us = timed(lambda i: ops.moe_combine(eos[i % n_e], row_of, wts, top, None, None, y, rows, residual=y))
        out["combine_" + label]["kuvusun"] = bytes_point(us, rows * width * (4 * top + 8))
        del eos
        # -- the gate on the merged heads: a logit per head beside a logit per column ---------------------------------------
        merged = torch.randn(rows, H * vdim, device=dev).to(bf)
        gl = torch.randn(rows, H * vdim, device=dev)
        us = timed(lambda i: ops.gate_mul(gl[:, :H], merged, merged, "sigmoid", rows, H * vdim, per=vdim))
        out["head_gate_" + label] = {"rakelorn": bytes_point(us, rows * H * vdim * 4)}
        us = timed(lambda i: ops.gate_mul(gl, merged, merged, "sigmoid", rows, H * vdim))
        out["head_gate_" + label]["kuvusun"] = bytes_point(us, rows * H * vdim * 8)
        # -- an expert's first product and its activation: up + relu² beside gate+up + silu·up, rows dealt evenly -----------------
        ff = z["expert_ff"]
        P = rows * top
        x = torch.randn(P, width, device=dev).to(bf)
        offs = i32([P * e // E for e in range(E + 1)])
        w1 = (torch.randn(E, ff, width, device=dev) * 0.02).to(bf)
        w2 = (torch.randn(E, 2 * ff, width, device=dev) * 0.02).to(bf)
        u2 = torch.zeros(P, 2 * ff, dtype=bf, device=dev)
        a = torch.zeros(P, ff, dtype=bf, device=dev)
        us = timed(lambda i: ops.linear_grouped(x, w1, a, offs, P, act="relu2"))       # (the activation in the product's epilogue)
        fl = 2.0 * P * ff * width
        out["expert_in_" + label] = {"rakelorn": {"us": round(us, 1), "tflops": round(fl / us / 1e6, 1), "frac_tensor": round(fl / us / 1e6 / bf16_tflops, 3),
                                                  "gb_s": round(E * ff * width * 2 / us / 1e3, 1), "frac_hbm": round(E * ff * width * 2 / us / 1e3 / hbm_gbs, 3)}}
        us = timed(lambda i: (ops.linear_grouped(x, w2, u2, offs, P), ops.gate_mul(u2[:, :ff], u2[:, ff:], a, "silu", P, ff)))
        out["expert_in_" + label]["kuvusun"] = {"us": round(us, 1), "tflops": round(2 * fl / us / 1e6, 1), "frac_tensor": round(2 * fl / us / 1e6 / bf16_tflops, 3),
                                                "gb_s": round(E * 2 * ff * width * 2 / us / 1e3, 1), "frac_hbm": round(E * 2 * ff * width * 2 / us / 1e3 / hbm_gbs, 3)}
        del w1, w2
    return out


#: Suposun at two sizes that resemble a real model's layers, beside a Kuvusun of the same width, depth, heads, head sizes and
#: feed-forwards (its closest relative in the framework: the same block with the norm on the sublayers' outputs, the
#: embedding as head, dense and routed feed-forwards, a layer that reads another's cache).  Layers: attention over all
#: keys + dense; windowed attention with kept first keys, cap, sinks and gate + experts; attention reading the first
#: layer's keys + experts; windowed attention + experts.
SUPOSUN_SIZES = {
    "s": dict(DESIGN_SIZES["s"], kv_heads=4, window=512, keep=64, ff_gated=2816, buckets=65521),
    "m": dict(DESIGN_SIZES["m"], kv_heads=2, window=1024, keep=128, ff_gated=5632, buckets=65521),
}


def suposun_config(z: dict) -> dict:
    def att(kind, **more):
        m = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
             "rot": {"base": 1e6, "dims": z["rot"]}}
        m.update(more)
        return {"type": kind, "mixer": m}
    win = att("attention", softcap=30.0, mask={"size": z["window"], "keep_first": z["keep"]})
    win["mixer"]["rot"] = {"base": 1e6, "dims": z["rot"], "scaling": {"factor": 4.0, "original": 4096, "fast": 16.0, "slow": 2.0}}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"], "limit": 7.0}, "router": {"experts": z["experts"], "top": z["top"]}}
    layers = [dict(att("attention_2"), mlp={"kind": "dense", "ff": z["ff_gated"]}), dict(win, mlp=moe),
              dict(att("attention_2", kv_from=0), mlp=moe), dict(win, mlp=moe)]
    return {"architecture": "Suposun", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "logit_scale": 0.5,
            "embedding": {"scale": 1.0, "bigram": {"buckets": z["buckets"], "mul_prev": 1000003, "mul_cur": 31}}, "layers": layers}


def suposun_kernels(z: dict, hbm_gbs: float, bf16_tflops: float) -> dict:
    """Suposun's own kernels alone, each beside the like kernel of a model that was there (20 launches replayed as one graph,
    inputs rotated over more than L2): attention with cap, kept first keys and sinks beside the same kernel with a plain
    window (Kotisun's), in a prompt step and in a decode step; the preparation of queries and keys with their norm beside
    the one without; the router by sigmoid scores beside Rakelorn's by a softmax; the experts' bounded gate beside
    Kuvusun's; the dense feed-forward's GELU gate beside Kotisun's relu gate; the embedding with its bigram row beside
    Kotisun's scaled embedding."""
    import types
    import torch
    from vlrf_b200.csrc import ops
    from vlrf_b200.parts.context import Workspace
    dev, bf = "cuda", torch.bfloat16
    width, H, G, dk = z["width"], z["heads"], z["kv_heads"], z["dim"]
    window, keep = z["window"], z["keep"]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)   # noqa: E731

    def timed(fn, reps=20):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(reps):
                fn(i)
        graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3

    def bytes_point(us, nbytes):
        return {"us": round(us, 1), "gb_s": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / hbm_gbs, 3), "mib": round(nbytes / 2**20, 1)}

    def flops_point(us, fl):
        return {"us": round(us, 1), "tflops": round(fl / us / 1e6, 1), "frac_tensor": round(fl / us / 1e6 / bf16_tflops, 4)}

    warm = torch.zeros(4096, 4096, device=dev)
    t_end = time.time() + 0.2
    while time.time() < t_end:
        warm.add_(1.0)
        torch.cuda.synchronize()
    del warm
    out = {}
    S, L, B = 2, 1024, 64
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    sink = torch.randn(H, device=dev)
    # -- attention over a paged cache whose blocks are dealt at random; several caches, so that a launch finds none in L2 -----
    for label, n_seq, n_new, ctx_len in (("prompt", S, L, L), ("decode", B, 1, L)):
        blocks_per = (ctx_len + 63) // 64
        nb = n_seq * blocks_per
        per_cache = nb * G * 64 * dk * 2 * 2
        n_c = max(2, int(300e6 // per_cache) + 1) if label == "decode" else 2
        caches = [(torch.randn(nb, G, 64, dk, device=dev).to(bf), torch.randn(nb, G, 64, dk, device=dev).to(bf)) for _ in range(n_c)]
        table = torch.randperm(nb, device=dev).to(torch.int32).view(n_seq, blocks_per).contiguous()
        T = n_seq * n_new
        q = torch.randn(T, H * dk, device=dev).to(bf)
        o = torch.zeros(T, H * dk, dtype=bf, device=dev)
        c = types.SimpleNamespace(n_tokens=T, n_seqs=n_seq, max_new=n_new, max_context=ctx_len, ws=Workspace(dev), dev_err=err,
                                  seq_slot=i32(list(range(n_seq))), seq_start=i32([i * n_new for i in range(n_seq + 1)]),
                                  seq_pos0=i32([ctx_len - n_new] * n_seq), tok_slot=i32([s for s in range(n_seq) for _ in range(n_new)]),
                                  tok_pos=i32([ctx_len - n_new + j for _ in range(n_seq) for j in range(n_new)]))
        run = lambda i, **kw: ops.attention_window_step(q, caches[i % n_c][0], caches[i % n_c][1], table, o, c, H, G, dk, dk, dk ** -0.5, window, 1.0, **kw)  # noqa: E731
        us_new = timed(lambda i: run(i, softcap=30.0, keep_first=keep, sink=sink))
        us_old = timed(lambda i: run(i))
        if label == "decode":
            seen_new, seen_old = min(ctx_len, window + keep), min(ctx_len, window)
            out["attention_decode"] = {"suposun": bytes_point(us_new, n_seq * G * seen_new * dk * 4),
                                       "plain_window": bytes_point(us_old, n_seq * G * seen_old * dk * 4)}
        else:
            def pairs(extra):       # (query, key) pairs a head computes: the window's, and the kept keys where the window has left them
                return sum(min(p + 1, window) + (min(extra, max(0, p + 1 - window)) if extra else 0) for p in range(n_new))
            out["attention_prompt"] = {"suposun": flops_point(us_new, 4.0 * n_seq * H * dk * pairs(keep)),
                                       "plain_window": flops_point(us_old, 4.0 * n_seq * H * dk * pairs(0))}
        del caches
    pctx = types.SimpleNamespace(n_tokens=S * L, n_seqs=S, seq_start=i32([0, L, 2 * L]), tok_slot=i32([s for s in range(S) for _ in range(L)]),
                                 tok_pos=i32(list(range(L)) * S), dev_err=err)
    dctx = types.SimpleNamespace(n_tokens=B, n_seqs=B, seq_start=i32(list(range(B + 1))), tok_slot=i32(list(range(B))), tok_pos=i32([L] * B), dev_err=err)
    for label, c, rows in (("prompt", pctx, S * L), ("decode", dctx, B)):
        # -- queries and keys: norm per head + rotation of neighbours + append, beside rotation + append ------------------------
        in_w = H * dk + G * dk + H
        n_p = max(2, int(300e6 // (rows * in_w * 4)) + 1)
        projs = [torch.randn(rows, in_w, device=dev) for _ in range(n_p)]
        nbk = max(S, B) * ((L + 64) // 64 + 1)
        kc, vc = torch.zeros(nbk, G, 64, dk, dtype=bf, device=dev), torch.zeros(nbk, G, 64, dk, dtype=bf, device=dev)
        table = torch.arange(nbk, dtype=torch.int32, device=dev).view(max(S, B), -1).contiguous()
        qo = torch.zeros(rows, H * dk, dtype=bf, device=dev)
        freq = torch.tensor([1e6 ** (-2.0 * i / z["rot"]) for i in range(z["rot"] // 2)], device=dev)
        wn = torch.ones(dk, device=dev)
        moved = rows * (in_w - H) * 4 + rows * (H + 2 * G) * dk * 2
        us = timed(lambda i: ops.qkv_rope_append(projs[i % n_p], 0, H * dk, H * dk, freq, z["rot"], qo, kc, vc, table, c.tok_slot, c.tok_pos, rows, H, G,
                                                 dk, dk, True, err, norm="head", q_norm=wn, k_norm=wn, eps=1e-6, interleaved=True, magnitude=1.2))
        out["prepare_" + label] = {"suposun": bytes_point(us, moved)}
        us = timed(lambda i: ops.qkv_rope_append(projs[i % n_p], 0, H * dk, H * dk, freq, z["rot"], qo, kc, vc, table, c.tok_slot, c.tok_pos, rows, H, G,
                                                 dk, dk, True, err))
        out["prepare_" + label]["without_norm"] = bytes_point(us, moved)
        del projs
        # -- the router: sigmoid scores with a correction beside a softmax over all outputs with one -------------------------
        E, top = z["experts"], z["top"]
        zl = torch.randn(rows, E, device=dev)
        ids = torch.zeros(rows, top, dtype=torch.int32, device=dev)
        rank = torch.zeros_like(ids)
        wts = torch.zeros(rows, top, device=dev)
        counts = torch.zeros(E, dtype=torch.int32, device=dev)
        corr = torch.zeros(E, device=dev)
        us0 = timed(lambda i: counts.zero_())
        us = timed(lambda i: (counts.zero_(), ops.moe_route_scored(zl, E, top, 1, 1, 0, 1.0, corr, None, ids, wts, rank, counts, rows, scoring="sigmoid")))
        out["router_" + label] = {"suposun": {"us": round(us - us0, 1)}}
        us = timed(lambda i: (counts.zero_(), ops.moe_route_scored(zl, E, top, 1, 1, 0, 1.0, corr, None, ids, wts, rank, counts, rows)))
        out["router_" + label]["softmax_all"] = {"us": round(us - us0, 1)}
        # -- the experts' gate: bounded beside x·sigmoid(x) ------------------------------------------------------------------
        ff, P = z["expert_ff"], rows * top
        n_u = max(2, int(300e6 // (P * 2 * ff * 2)) + 1)
        us_ = [torch.randn(P, 2 * ff, device=dev).to(bf) for _ in range(n_u)]
        a = torch.zeros(P, ff, dtype=bf, device=dev)
        us = timed(lambda i: ops.gate_mul_clamped(us_[i % n_u][:, :ff], us_[i % n_u][:, ff:], a, 7.0, 1.702, P, ff))
        out["expert_gate_" + label] = {"suposun": bytes_point(us, P * ff * 6)}
        us = timed(lambda i: ops.gate_mul(us_[i % n_u][:, :ff], us_[i % n_u][:, ff:], a, "silu", P, ff))
        out["expert_gate_" + label]["silu"] = bytes_point(us, P * ff * 6)
        del us_
        # -- the dense feed-forward's gate on float32 products: tanh GELU beside relu ------------------------------------------
        ffg = z["ff_gated"]
        n_g = max(2, int(300e6 // (rows * 2 * ffg * 4)) + 1)
        gus = [torch.randn(rows, 2 * ffg, device=dev) for _ in range(n_g)]
        u = torch.zeros(rows, ffg, dtype=bf, device=dev)
        us = timed(lambda i: ops.gate_mul(gus[i % n_g][:, :ffg], gus[i % n_g][:, ffg:], u, "gelu_tanh", rows, ffg))
        out["dense_gate_" + label] = {"suposun": bytes_point(us, rows * ffg * 10)}
        us = timed(lambda i: ops.gate_mul(gus[i % n_g][:, :ffg], gus[i % n_g][:, ffg:], u, "relu", rows, ffg))
        out["dense_gate_" + label]["relu"] = bytes_point(us, rows * ffg * 10)
        del gus
        # -- the embedding with its bigram row beside a scaled embedding -------------------------------------------------------
        V, buckets = z["vocab"], z["buckets"]
        table_e, pairs_t = torch.randn(V, width, device=dev).to(bf), torch.randn(buckets + 1, width, device=dev).to(bf)
        kept = torch.zeros(max(S, B), 2, dtype=torch.int32, device=dev)
        toks = [torch.randint(0, V, (rows,), dtype=torch.int32, device=dev) for _ in range(4)]
        x = torch.zeros(rows, width, device=dev)

        def emb(i):
            c.tokens = toks[i % 4]
            ops.embed_bigram(table_e, pairs_t, buckets, 1000003, 31, 1.0, kept, c, x)
        us = timed(emb)
        out["embed_" + label] = {"suposun": bytes_point(us, rows * width * 8)}
        us = timed(lambda i: ops.embed_streams(table_e, toks[i % 4], x, 1, 2.0, err))
        out["embed_" + label]["scaled"] = bytes_point(us, rows * width * 6)
        del table_e, pairs_t
    return out


def design_bench(args) -> int:
    """`--design NAME`: the design at sizes like a real model's layers (random weights) beside its closest existing
    model of equal size (GPT-2; for Rakelorn, Kuvusun): prefill and decode throughput, and each kernel's time.  One JSON line."""
    import vlrf_b200.models  # noqa: F401
    from vlrf_b200.weights import write_random_model
    hbm_gbs, bf16_tflops, peak_src = peaks()
    line = {"design": args.design, "beside": "gpt2", "dtype": "bf16", "data": "synthetic (seeded random token ids, random weights)",
            "peaks": {"hbm_gbs": hbm_gbs, "bf16_tflops": bf16_tflops, "source": peak_src}, "sizes": {}}
    sizes, config_of, kernels_of = {"kuvusun": (DESIGN_SIZES, kuvusun_config, design_kernels),
                                    "kotisun": (KOTISUN_SIZES, kotisun_config, kotisun_kernels),
                                    "rakelorn": (RAKELORN_SIZES, rakelorn_config, rakelorn_kernels),
                                    "suposun": (SUPOSUN_SIZES, suposun_config, suposun_kernels)}[args.design]
    beside, beside_of = {"rakelorn": ("kuvusun", kuvusun_config_like), "suposun": ("kuvusun", kuvusun_config)}.get(args.design, ("gpt2", gpt2_config_like))
    line["beside"] = beside
    for name in args.design_sizes.split(","):
        z = sizes[name]
        point = {"sizes": z}
        with tempfile.TemporaryDirectory(prefix="vlrf_b200_bench_") as tmp:
            for label, cfg in (() if args.design_only_kernels else ((args.design, config_of(z)), (beside, beside_of(z)))):
                d = str(write_random_model(cfg, 1234, os.path.join(tmp, label)))
                point[label] = design_point(d, args.design_prompt, [8, 64], max(8, min(args.steps, 64)), max(3, min(args.warmup, 8)))
        if not args.design_no_kernels:
            point["kernels"] = kernels_of(z, hbm_gbs, bf16_tflops)
        line["sizes"][name] = point
    print(json.dumps(line))
    return 0



def metric_label(preset: str, batch: int, first_context: int, last_context: int) -> str:
    sizes = "GPT-2 small sizes" if preset == "gpt2" else preset
    return f"decode tokens/s ({sizes}, batch {batch}, contexts {first_context} to {last_context})"


def reference_arm(args) -> int:
    """`--impl reference`: the unmodified reference, built from baseline/_ref by its own CMakeLists.txt and driven
    through its C API by baseline/reference_arm.py in a process of its own (nothing of this package is loaded
    there).  It prints the same JSON line, or an `unavailable` line that says why."""
    if args.gpus != 1:
        print(f"bench.py measures one GPU: the reference runs on the host cores (asked for --gpus {args.gpus})")
        return 2
    warmup = max(3, args.warmup)
    steps = min(args.steps, 1024 - PROMPT_LEN - warmup - 2)
    cmd = [sys.executable, os.path.join(ROOT, "baseline", "reference_arm.py"), "--steps", str(steps), "--warmup",
           str(warmup), "--batch", str(args.batch)]
    if args.layers is not None:
        cmd += ["--layers", str(args.layers)]
    try:
        done = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, timeout=900)
        lines = [ln for ln in done.stdout.splitlines() if ln.startswith("{")]
        line = json.loads(lines[-1])
    except (OSError, subprocess.TimeoutExpired, IndexError, ValueError) as e:
        line = {"impl": "reference", "unavailable": f"the reference's harness gave no result ({type(e).__name__})"}
    if "unavailable" not in line:
        line["metric"] = metric_label("gpt2", args.batch, PROMPT_LEN + warmup, PROMPT_LEN + warmup + steps)
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=496, help="decode steps to time (496 after 16 warm-up steps ends at position 1,024)")
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--preset", default="gpt2")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the preset (named in config)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--timeline", action="store_true",
                    help="with --only decode or prefill and VLRF_B200_KERNEL_TRACE=1: print where the last step's kernels spent their time")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="measure one part only and print a short line (for profiling runs); the full line needs 'all'")
    ap.add_argument("--design", default=None, choices=["kuvusun", "kotisun", "rakelorn", "suposun"],
                    help="instead of the default workload: this design at sizes like a real model's layers beside its closest "
                         "existing model of equal size (GPT-2; for rakelorn and suposun, Kuvusun)")
    ap.add_argument("--design-sizes", default="s,m", help="with --design: which of the sizes %s" % ",".join(DESIGN_SIZES))
    ap.add_argument("--design-no-kernels", action="store_true", help="with --design: whole steps only, not each kernel alone")
    ap.add_argument("--design-only-kernels", action="store_true", help="with --design: each kernel alone only")
    ap.add_argument("--design-prompt", type=int, default=1024, help="with --design: tokens of each of the two prompts, and the decode steps' first context")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.design is not None:
        return design_bench(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library has no multi-GPU path (asked for --gpus {args.gpus})")
        return 2
    warmup = max(3, args.warmup)

    import torch
    from vlrf_b200.config import load_preset
    hbm_gbs, bf16_tflops, peak_src = peaks()
    full_layers = load_preset(args.preset)["n_layer"]
    with tempfile.TemporaryDirectory(prefix="vlrf_b200_bench_") as tmp:
        model_dir = make_model_dir(args.preset, args.layers, tmp)
        if args.only == "decode":
            dec = decode_device(model_dir, args.batch, args.steps, warmup)
            print(json.dumps({"only": "decode", "batch": args.batch, "tok_s": round(dec["tok_s"], 1),
                              "ms_per_step": round(dec["ms_per_step"], 4), "kernels_per_step": dec["kernels_per_step"]}))
            if args.timeline:
                from vlrf_b200 import log
                print(log.timeline_table(log.kernel_timeline(), last=5 * dec["n_layer"]))
            return 0
        if args.only == "prefill":
            pre = prefill_device(model_dir, reps=max(1, args.steps))
            print(json.dumps({"only": "prefill", "tokens": pre["tokens"], "ms": round(pre["ms"], 4)}))
            if args.timeline:
                from vlrf_b200 import log
                print(log.timeline_table(log.kernel_timeline(), last=5 * full_layers if args.layers is None else 5 * args.layers))
            return 0
        dec = decode_device(model_dir, args.batch, args.steps, warmup)
        e2e = decode_e2e(model_dir, args.batch, dec["steps"], warmup)
        pre = prefill_device(model_dir)
        pre_new_shape = prefill_device(model_dir, replay=False)
        points = {}
        if not args.skip_points:
            for b in (1, 64):
                points[f"decode_b{b}"] = round(decode_device(model_dir, b, min(args.steps, 128), warmup)["tok_s"], 1)
    if not args.skip_points and args.preset == "gpt2" and args.layers is None:
        # the largest size of the family at its full depth, where a step is bound by bytes rather than by latencies
        with tempfile.TemporaryDirectory(prefix="vlrf_b200_bench_") as tmp:
            xl = decode_device(make_model_dir("gpt2-xl", None, tmp), 8, 64, warmup)
        points["xl_decode_b8"] = round(xl["tok_s"], 1)
        points["xl_decode_b8_hbm_frac"] = round(xl["bytes_per_step"] / (xl["ms_per_step"] / 1e3) / 1e9 / hbm_gbs, 4)
    cfg = load_preset(args.preset)
    achieved = dec["bytes_per_step"] / (dec["ms_per_step"] / 1e3) / 1e9
    pre_tflops = pre["flops"] / (pre["ms"] / 1e3) / 1e12
    line = {
        "metric": metric_label(args.preset, args.batch, PROMPT_LEN + warmup, PROMPT_LEN + warmup + dec["steps"]),
        "value": round(dec["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": dec["steps"], "warmup": warmup,
        "ms_per_step": round(dec["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded random token ids, random weights)",
        "impl": "ours",
        "config": {
            "model": args.preset, "n_layer": dec["n_layer"], "n_layer_of_config": full_layers,
            "n_embd": cfg["n_embd"], "n_head": cfg["n_head"], "n_inner": cfg["n_inner"] or 4 * cfg["n_embd"],
            "vocab_size": cfg["vocab_size"], "n_positions": cfg["n_positions"], "global_batch": args.batch,
            "seq_len": cfg["n_positions"], "prompt_len": PROMPT_LEN, "mean_context": dec["mean_context"],
            "parallelism": "single GPU", "weights": "bf16 random", "kv_cache": "bf16 paged, 64-token blocks",
            "l2": "working set of a step exceeds L2; no flush", "peaks": peak_src,
            "kernels_per_step": dec["kernels_per_step"],
        },
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d"],
                "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": dec["launches"],
        "prefill": {"value": round(pre["tokens"] / (pre["ms"] / 1e3), 1), "tokens": pre["tokens"],
                    "ms": round(pre["ms"], 4), "frac": round(pre_tflops / bf16_tflops, 4),
                    "ms_new_shape": round(pre_new_shape["ms"], 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4)},
        "points": points,
        "clocks": dec["clocks"],
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
