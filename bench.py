#!/usr/bin/env python
"""Token-loop benchmark: batch-1 decode tok/s (headline) and prefill tok/s on a seeded synthetic model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config NAME]

One step = one pass of the workload: roll the sequence back to 0, evaluate the prompt (prefill), then decode
greedily. `value` is decode tokens/s with everything resident in HBM (on-device greedy loop, CUDA-event time);
`e2e` is the same metric through the Engine-shaped public call with host buffers: token ids copied in and all
logits copied out every step, arg-max on the host - the loop brisk-llm's `generate` runs. With N > 1 every rank
runs an independent replica (batch-1 decode of one sequence has nothing to shard for this configuration).
After the headline the same run times the one configuration that does shard - the Mistral-7B-shaped Q4_0 model,
8192-token prompt + 512 greedy steps - tensor-parallel over all N ranks (N = 1: on the one GPU) and reports it in the
`tensor_parallel` object, so the 1 -> N scaling of that configuration can be read from the per-N lines.
`--impl reference` times the reference's own CPU engine on the host cores instead.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from brisk_llm_b200 import formats as F, synth  # noqa: E402

METRIC = "decode_tokens_per_s_batch1"
UNIT = "tok/s"
FALLBACK_HBM_GBS = 6650.0


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=5)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--config", default="qwen3-0.6b-q4_0", choices=sorted(synth.PRESETS))
    p.add_argument("--prompt", type=int, default=0)
    p.add_argument("--decode", type=int, default=0)
    p.add_argument("--layers", type=int, default=0, help="override the layer count (debugging; the reported number is then not the configured workload)")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-tp", action="store_true", help="skip the tensor-parallel section (the 7B-shaped configuration)")
    p.add_argument("--spec", type=int, default=0, metavar="D", help="instead of the headline: the speculative-verify variant of the 7B-shaped configuration - "
                   "4 sequences, D drafted tokens per verify step (n-gram lookup drafts), on one GPU")
    p.add_argument("--profile", action="store_true", help="for ncu launch lists: exactly --warmup warm-up steps, no end-to-end loop, no CPU baseline (the printed number is not a bench value)")
    return p.parse_args()


WORKLOADS = {  # prompt tokens, decode steps, context
    "qwen3-0.6b-q4_0": (512, 128, 2048),
    "llama-3.2-1b-q4_k_m": (1024, 256, 4096),
    "bitnet-2b4t-tq2_0": (512, 256, 4096),
    "mistral-7b-q4_0": (8192, 512, 8704),
    "gemma3-1b-q4_0": (1024, 256, 4096),  # not a benchmark configuration: the Gemma 3 layer variants at a real model's shape
}


def analytic_traffic(spec, weight_bytes, prompt, decode):
    """DRAM bytes one decoded token must move, counted (not measured): every weight plane once, the visible K/V cache at
    the mean context of the decode steps, the logits row written. ncu's dram__bytes of the token kernel at context ~516
    (profiles/) agrees with this figure to a few percent; the number here follows the workload, not a capture."""
    mean_ctx = prompt + decode / 2
    kv = spec.layers * 2 * spec.kv_heads * spec.head_dim * 2 * mean_ctx
    return int(weight_bytes + kv + spec.vocab * 4)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines, self.t0 = index, None, [], None

    def mark(self):
        """The timed region starts now: samples from here on are the ones reported (the sampler itself is started a warm-up
        step earlier - with eight ranks starting nvidia-smi at once its first line can take longer than a short timed region)."""
        self.t0 = time.perf_counter()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [line for t, line in self.lines if self.t0 is None or t >= self.t0]
        window = "timed region"
        if not inside:  # a timed region shorter than the sampling period: the warm-up step before it ran the same load
            inside, window = [line for _, line in self.lines], "last warm-up step and timed region"
        for line in inside:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


def workload_for(args):
    spec = synth.PRESETS[args.config]
    prompt, decode, ctx = WORKLOADS[args.config]
    prompt = args.prompt or prompt
    decode = args.decode or decode
    if args.layers:
        from dataclasses import replace
        spec = replace(spec, layers=args.layers)
    from dataclasses import replace
    spec = replace(spec, context=ctx)
    return spec, prompt, decode


def describe(spec, prompt, decode, extra=None):
    cfg = {"workload": f"{spec.name}: {spec.layers} layers, hidden {spec.hidden}, {spec.heads}/{spec.kv_heads} heads x {spec.head_dim}, "
                       f"ffn {spec.ffn}, vocab {spec.vocab}, {F.NAMES[spec.fmt]}; {prompt}-token random prompt + {decode} greedy decode "
                       f"steps, batch 1, f16 K/V cache, ctx {spec.context}",
           "l2": "every token streams all weight planes, larger than the 126 MB L2, so timed iterations do not reuse cached inputs",
           "weights": "seeded synthetic, f32 N(0,0.02) quantised (no checkpoint available)"}
    if extra:
        cfg.update(extra)
    return cfg


# ---- reference / CPU arm ------------------------------------------------------------------------------------------

def cpu_engine(model, spec, threads):
    """The reference CPU engine (oracle/_ref, built from a reference checkout) when it is present, else the C port."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import helpers as H
    if H.have_ref():
        from brisk_llm_b200 import gguf_io
        path = os.path.join(tempfile.gettempdir(), f"brisk_bench_{spec.name}_{spec.layers}_{os.getpid()}.gguf")
        gguf_io.write_gguf(model, path)
        r = H.ref()
        handle = r.ref_session_create(path.encode(), threads, spec.context)
        if not handle:
            raise RuntimeError(r.ref_last_error().decode())

        def run(prompt_ids, steps, want_logits=False):
            r.ref_session_rollback(handle, 0)
            out = np.empty(steps, np.int32)
            logits = np.empty((steps, spec.vocab), np.float32) if want_logits else None
            tp, td = C.c_double(), C.c_double()
            rc = r.ref_session_generate_greedy(handle, H.iptr(prompt_ids), len(prompt_ids), steps, H.iptr(out),
                                               H.fptr(logits) if want_logits else None, C.byref(tp), C.byref(td))
            if rc != 0:
                raise RuntimeError(r.ref_last_error().decode())
            return (tp.value, td.value, out, logits) if want_logits else (tp.value, td.value)

        def close():
            r.ref_session_destroy(handle)
            os.remove(path)

        return "reference", r.ref_kernel_set_name().decode(), run, close
    os.environ["BRISK_ORACLE_THREADS"] = str(threads)
    sess = H.OracleSession(model, spec.context)

    def run(prompt_ids, steps, want_logits=False):
        sess.rollback(0)
        rows, picks = [], []
        t0 = time.perf_counter()
        logits = sess.eval(prompt_ids)
        t1 = time.perf_counter()
        for i in range(steps):
            if want_logits:
                rows.append(logits.copy())
            picks.append(int(np.argmax(logits)))
            if i + 1 < steps:
                logits = sess.eval([picks[-1]])
        t2 = time.perf_counter()
        return (t1 - t0, t2 - t1, np.array(picks, np.int32), np.stack(rows)) if want_logits else (t1 - t0, t2 - t1)

    return "port", "scalar C port", run, sess.close


def cpu_sample_sizes(spec, prompt, decode):
    """(prompt tokens, greedy picks) of one CPU step. The 0.6B-class configuration runs its whole workload (about 10-20 s on
    a few dozen cores; `decode` + 1 picks are `decode` decoded tokens); larger models a sample whose cost stays in that
    range - it shrinks with the weight bytes per token."""
    scale = spec.layers * (spec.hidden * (spec.q_dim * 2 + spec.kv_dim * 2 + 3 * spec.ffn)) / 4.4e8
    if scale <= 1.05:
        return prompt, decode + 1
    return max(8, int(128 / scale)), max(4, int(32 / scale))


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    spec, prompt, decode = workload_for(args)
    model = synth.generate(spec, seed=0, share_layers=spec.layers * spec.hidden * spec.ffn > 1e9)
    threads = os.cpu_count() or 1
    sp, sd = cpu_sample_sizes(spec, prompt, decode)
    kind, kernels, run, close = cpu_engine(model, spec, threads)
    ids = synth.random_tokens(spec, sp, seed=1)
    # a CPU step is ten seconds or more: at most three timed steps and one warm-up, whatever was asked for, so that the
    # whole run ends within a few minutes
    steps, warmup = min(args.steps, 3), min(args.warmup, 1)
    for _ in range(warmup):
        run(ids, sd)
    tp = td = 0.0
    for _ in range(steps):
        a, b = run(ids, sd)
        tp += a
        td += b
    close()
    value = steps * (sd - 1) / td if td > 0 else 0.0
    whole = (sp, sd - 1) == (prompt, decode)
    sample = (f"the whole workload ({sp}-token prompt + {sd - 1} decoded tokens) per step, {steps} timed steps" if whole else
              f"{sp}-token prompt + {sd - 1} decoded tokens of the same model per step, {steps} timed steps") + f" ({kernels} kernels)"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": warmup, "ms_per_step": 1e3 * (tp + td) / steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 dot products, f32 accumulate", "data": "synthetic",
            "config": describe(spec, prompt, decode, {"sample": sample, "same_workload": whole}), "prefill_tokens_per_s": steps * sp / tp,
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---- our arm ------------------------------------------------------------------------------------------------------

def tensor_parallel_section(engine, torch, dist, rank, local, world, max_over_ranks, barrier):
    """The configuration that shards: the Mistral-7B-shaped Q4_0 model, 8192-token prompt filling the f16 K/V cache, then
    512 greedy steps, batch 1 - on one GPU, or tensor-parallel over all ranks (every matrix split by output rows, K/V
    heads split, activations exchanged inside the library). One warm-up pass (prompt + 16 steps), one timed pass; device
    time by CUDA events on the session's stream, maximum over the ranks."""
    from dataclasses import replace
    from brisk_llm_b200 import parallel
    prompt, decode, ctx = WORKLOADS["mistral-7b-q4_0"]
    spec = replace(synth.PRESETS["mistral-7b-q4_0"], context=ctx)
    model = synth.generate(spec, seed=0, share_layers=True)  # one layer's weights drawn, reused by all 32 (same shapes and distributions)
    ids = synth.random_tokens(spec, prompt, seed=1)
    sess = parallel.tensor_parallel_session(model, max_context=ctx) if world > 1 else engine.CudaSession(model, max_context=ctx, device=local)
    try:
        def one_pass(steps):
            sess.rollback(0)
            logits = sess.eval(ids)
            pre = sess.stats()["device_ms"]
            sess.generate_greedy(int(np.argmax(logits)), steps)
            return pre, sess.stats()["device_ms"]
        one_pass(16)
        barrier()
        pre_ms, dec_ms = one_pass(decode)
        barrier()
        # share of a decode step spent exchanging activations: per-phase device time of 16 more steps (profiling runs the
        # step kernel by kernel, so this is a share, not a speed)
        sess.rollback(prompt)
        sess.profile(True)
        sess.generate_greedy(0, 16)
        phases = sess.profile(False)
        total = sum(v["ms"] for v in phases.values())
        exchange = phases.get("exchange", {"ms": 0.0})["ms"] / total if total > 0 else 0.0
        pre_ms, dec_ms = max_over_ranks(pre_ms), max_over_ranks(dec_ms)
        weight_bytes = model.weight_bytes()
        peak, peak_kind = peaks()
        per_gpu = weight_bytes / world * decode / (dec_ms * 1e-3) / 1e9
        return {"config": f"{spec.name}: {spec.layers} layers, hidden {spec.hidden}, {spec.heads}/{spec.kv_heads} heads x {spec.head_dim}, ffn {spec.ffn}, "
                          f"vocab {spec.vocab}, Q4_0; {prompt}-token random prompt + {decode} greedy decode steps, batch 1, f16 K/V cache, ctx {ctx}",
                "tp": world, "parallelism": "single GPU" if world == 1 else f"tensor parallel x{world}: matrices split by output rows, K/V heads split",
                "decode_tokens_per_s": decode / (dec_ms * 1e-3), "decode_us_per_token": 1e3 * dec_ms / decode,
                "prefill_tokens_per_s": prompt / (pre_ms * 1e-3), "scaling": "strong",
                "roofline_frac_per_gpu": per_gpu / peak, "roofline_achieved_gbs_per_gpu": per_gpu, "peak_kind": f"of {peak_kind}",
                "exchange_share_of_decode_step": exchange, "single_token_path": sess.step_path()}
    finally:
        sess.close()


def run_speculative(args):
    """configs[4]'s second workload: 4 sequences of the Mistral-7B-shaped model, each an 8192-token prompt, then 512 tokens
    settled by lookup-draft speculative decoding with D drafted tokens per verify step (Speculator + LookupDrafter,
    brisk-llm src/speculative.cpp:45-118: a verify step is eval_all(1 + drafts) and a rollback). The four sessions are
    stepped round-robin from one host thread, every call with host buffers (the logits of all 1 + D rows come back)."""
    import torch  # noqa: F401  (device initialisation order as in the main arm)
    from dataclasses import replace
    from brisk_llm_b200 import engine, speculative
    prompt_len, decode, ctx = WORKLOADS["mistral-7b-q4_0"]
    prompt_len, decode = args.prompt or prompt_len, args.decode or decode
    ctx += 64  # a verify step evaluates up to D tokens past the last settled one: room for it at the end of the run
    spec = replace(synth.PRESETS["mistral-7b-q4_0"], context=ctx)
    model = synth.generate(spec, seed=0, share_layers=True)
    sequences = 4
    sessions = [engine.CudaSession(model, max_context=ctx) for _ in range(sequences)]
    try:
        # text that repeats itself, so that the drafter has something to propose: a 64-token motif with seeded variations
        rng = np.random.default_rng(1)
        prompts = []
        for i in range(sequences):
            motif = rng.integers(0, spec.vocab, size=64, dtype=np.int32)
            prompts.append(np.tile(motif, prompt_len // 64 + 1)[:prompt_len].copy())
        t0 = time.perf_counter()
        specs = []
        for sess, prm in zip(sessions, prompts):
            drafter = speculative.LookupDrafter()
            drafter.observe(prm)
            sess.eval(prm[:-1])
            specs.append(speculative.Speculator(sess, drafter, int(prm[-1]), args.spec))
        t_prefill = time.perf_counter() - t0
        settled = [0] * sequences
        verify_ms, plain_ms, verify_n, plain_n = 0.0, 0.0, 0, 0
        by_tokens = {}  # tokens in the verify step (1 + its drafts) -> [steps, device ms]
        t0 = time.perf_counter()
        while min(settled) < decode:
            for i, sp in enumerate(specs):
                if settled[i] >= decode:
                    continue
                was_plain = sp.backoff > 0
                drafted_before = sp.stats["drafted"]
                settled[i] += len(sp.step())
                ms = sessions[i].stats()["device_ms"]
                if was_plain:
                    plain_ms, plain_n = plain_ms + ms, plain_n + 1
                else:
                    verify_ms, verify_n = verify_ms + ms, verify_n + 1
                    slot = by_tokens.setdefault(1 + sp.stats["drafted"] - drafted_before, [0, 0.0])
                    slot[0], slot[1] = slot[0] + 1, slot[1] + ms
        wall = time.perf_counter() - t0
        stats = {k: sum(sp.stats[k] for sp in specs) for k in specs[0].stats}
        # the verify step by itself, at the context the run ended on: eval_all of 1 + D tokens and the rollback, against one token
        sess, pos = sessions[0], sessions[0].position()
        probe = rng.integers(0, spec.vocab, size=1 + args.spec, dtype=np.int32)
        full_ms = one_ms = 0.0
        reps = 10
        for r in range(reps + 2):
            sess.eval_all(probe)
            a = sess.stats()["device_ms"]
            sess.rollback(pos)
            sess.eval(probe[:1])
            b = sess.stats()["device_ms"]
            sess.rollback(pos)
            if r >= 2:
                full_ms, one_ms = full_ms + a / reps, one_ms + b / reps
        line = {"metric": "speculative_settled_tokens_per_s", "value": sum(settled) / wall, "unit": "tok/s", "n_gpus": 1, "higher_is_better": True,
                "data": "synthetic", "config": {"workload": f"{spec.name}: {sequences} sequences x ({prompt_len}-token repeating prompt + {decode} settled tokens), "
                                                            f"{args.spec} drafted tokens per verify step (n-gram lookup), ctx {ctx}, one GPU, host buffers"},
                "verify_steps": verify_n, "ms_per_verify_step_device": verify_ms / max(verify_n, 1), "plain_steps": plain_n,
                "ms_per_plain_step_device": plain_ms / max(plain_n, 1) if plain_n else None,
                "verify_step_over_plain_step": (verify_ms / max(verify_n, 1)) / (plain_ms / plain_n) if plain_n else None,
                "verify_steps_by_tokens": {str(k): {"steps": v[0], "ms_device": v[1] / v[0]} for k, v in sorted(by_tokens.items())},
                "probe": {"context": pos, "tokens": 1 + args.spec, "eval_all_ms_device": full_ms, "eval_one_ms_device": one_ms, "ratio": full_ms / one_ms},
                "drafted": stats["drafted"], "accepted": stats["accepted"], "prefill_tokens_per_s": sequences * (prompt_len - 1) / t_prefill,
                "wall_s": wall}
        print(json.dumps(line), flush=True)
    finally:
        for sess in sessions:
            sess.close()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.spec:
        run_speculative(args)
        return
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    # single node: NCCL's bootstrap must not depend on the container's host name resolving
    os.environ.setdefault("NCCL_SOCKET_IFNAME", "lo")
    os.environ.setdefault("NCCL_IB_DISABLE", "1")
    import torch
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from brisk_llm_b200 import engine

    spec, prompt, decode = workload_for(args)
    big = spec.layers * spec.hidden * spec.ffn > 1e9  # 7B-class: draw one layer's weights and reuse them (same shapes and distributions)
    model = synth.generate(spec, seed=0, share_layers=big)
    ids = synth.random_tokens(spec, prompt, seed=1)
    tensor_parallel = world > 1 and args.config == "mistral-7b-q4_0"
    if tensor_parallel:
        from brisk_llm_b200 import parallel
        sess = parallel.tensor_parallel_session(model, max_context=spec.context)
    else:
        sess = engine.CudaSession(model, max_context=spec.context, device=local)
    weight_bytes = model.weight_bytes()
    jobs = 1 if tensor_parallel else world  # sequences decoded at once by the whole job

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def device_step():
        sess.rollback(0)
        logits = sess.eval(ids)
        st = sess.stats()
        pre_ms, launches = st["device_ms"], st["kernel_launches"]
        first = int(np.argmax(logits))
        sess.generate_greedy(first, decode)
        st = sess.stats()
        return pre_ms, st["device_ms"], launches + st["kernel_launches"]

    def e2e_step():
        sess.rollback(0)
        h2d = d2h = 0
        t0 = time.perf_counter()
        logits = sess.eval(ids)
        st = sess.stats()
        h2d, d2h = h2d + st["h2d_bytes"], d2h + st["d2h_bytes"]
        t1 = time.perf_counter()
        for _ in range(decode):
            # the logits are read where the session leaves them (pinned host memory, valid until the next call -
            # the span Engine::eval returns), as the reference's sampler reads them
            logits = sess.eval([int(np.argmax(logits))], copy=False)
            st = sess.stats()
            h2d, d2h = h2d + st["h2d_bytes"], d2h + st["d2h_bytes"]
        t2 = time.perf_counter()
        return t1 - t0, t2 - t1, h2d, d2h

    def topk_step(k=20):
        """Decode through eval_topk: per token 4 bytes of token id in, k (id, logit) pairs out - what a sampling host needs
        (here it takes the first pair, so the sequence is the greedy one)."""
        sess.rollback(0)
        logits = sess.eval(ids)
        nxt = int(np.argmax(logits))
        t1 = time.perf_counter()
        for _ in range(decode):
            top_ids, _ = sess.eval_topk([nxt], k)
            nxt = int(top_ids[0])
        return time.perf_counter() - t1

    warmups = args.warmup if args.profile else max(args.warmup, 3)
    sampler = ClockSampler(local)
    for i in range(warmups):
        if i == warmups - 1:
            sampler.start()
        device_step()
    if sampler.proc is None:
        sampler.start()
    barrier()
    sampler.mark()
    pre_ms = dec_ms = 0.0
    launches = 0
    t_wall = time.perf_counter()
    for _ in range(args.steps):
        a, b, c = device_step()
        pre_ms, dec_ms, launches = pre_ms + a, dec_ms + b, launches + c
    barrier()
    t_wall = time.perf_counter() - t_wall
    clocks = sampler.stop()

    e_pre = e_dec = 1e-9
    h2d = d2h = 0
    if not args.profile:
        e2e_step()
        barrier()
        e_pre = e_dec = 0.0
        for _ in range(args.steps):
            a, b, c, d = e2e_step()
            e_pre, e_dec, h2d, d2h = e_pre + a, e_dec + b, c, d
        barrier()
        topk_step()
        k_dec = sum(topk_step() for _ in range(args.steps))
        barrier()

    def max_over_ranks(v):
        if dist is None:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    pre_ms, dec_ms, e_pre, e_dec = (max_over_ranks(v) for v in (pre_ms, dec_ms, e_pre, e_dec))
    k_dec = max_over_ranks(k_dec) if not args.profile else 0.0
    tp_line = None
    if not args.profile and not args.no_tp and args.config == "qwen3-0.6b-q4_0" and not args.layers:
        try:
            tp_line = tensor_parallel_section(engine, torch, dist, rank, local, world, max_over_ranks, barrier)
        except Exception as e:  # reported, never allowed to take the headline down with it
            tp_line = {"failed": f"{type(e).__name__}: {e}"}
    if rank == 0:
        peak, peak_kind = peaks()
        tokens = args.steps * decode
        value = jobs * tokens / (dec_ms * 1e-3)
        achieved = weight_bytes / (world if tensor_parallel else 1) * tokens / (dec_ms * 1e-3) / 1e9  # per GPU
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmups,
                "ms_per_step": (pre_ms + dec_ms) / args.steps, "higher_is_better": True, "scaling": "strong" if tensor_parallel else "weak",
                "vs_baseline": None,
                "dtype": "int8 dot products, f32 accumulate (f16 K/V cache)", "data": "synthetic",
                "config": describe(spec, prompt, decode, {"parallelism": f"tensor parallel x{world} (row-split matrices, all-gathers)" if tensor_parallel
                                                          else "replicas only" if world > 1 else "single GPU"}),
                "prefill_tokens_per_s": jobs * args.steps * prompt / (pre_ms * 1e-3),
                "decode_us_per_token": 1e3 * dec_ms / tokens,
                "wall_s_timed_region": t_wall,
                "e2e": {"value": jobs * tokens / e_dec, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "prefill_tokens_per_s": jobs * args.steps * prompt / e_pre},
                "e2e_topk": None if args.profile else {"value": jobs * args.steps * decode / k_dec, "unit": UNIT, "k": 20, "h2d_bytes_per_token": 8, "d2h_bytes_per_token": 160,
                                                       "note": "eval_topk per token: the host gets the 20 best (id, logit) pairs instead of the whole row"},
                "gpu_launches": launches,
                "clocks": clocks,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "traffic": analytic_traffic(spec, weight_bytes, prompt, decode) if world == 1 else None,
                             "traffic_kind": "analytic: weights + visible K/V at the mean context + logits (ncu captures under profiles/ agree)",
                             "peak_kind": f"of {peak_kind}", "kernel": "decode step (all kernels of one token)",
                             "algorithmic_bytes_per_token": weight_bytes // (world if tensor_parallel else 1)}}
        line["config"]["single_token_path"] = sess.step_path()
        if args.profile:
            line["profile_run"] = True
            line.pop("e2e")
        if world == 1 and not args.no_cpu_baseline and not args.profile:
            try:
                threads = os.cpu_count() or 1
                sp, sd = cpu_sample_sizes(spec, prompt, decode)
                kind, kernels, run, close = cpu_engine(model, spec, threads)
                cpu_ids = synth.random_tokens(spec, sp, seed=1)
                tp, td, want_picks, want_logits = run(cpu_ids, sd, want_logits=True)
                close()
                whole = (sp, sd - 1) == (prompt, decode)
                line["cpu_baseline"] = {"value": (sd - 1) / td, "unit": UNIT, "cores": threads, "kind": kind,
                                        "sample": ("the whole workload: " if whole else "") + f"{sp}-token prompt + {sd - 1} decoded tokens of the same model ({kernels} kernels)",
                                        "prefill_tokens_per_s": sp / tp}
                # parity on this very run: the device's logits for the CPU leg's prompt and picks against the CPU leg's own
                sess.rollback(0)
                first = sess.eval(cpu_ids)
                got_picks, got_logits = sess.generate_greedy(int(np.argmax(first)), sd - 1, want_logits=True)
                got = np.concatenate([first[None, :], got_logits])
                got_all = np.concatenate([[int(np.argmax(first))], got_picks])[:sd]
                diff = np.abs(got - want_logits)
                rel = max(float(np.linalg.norm((g - w).astype(np.float64)) / max(np.linalg.norm(w.astype(np.float64)), 1e-30)) for g, w in zip(got, want_logits))
                line["parity"] = {"against": kind, "rows": int(sd), "max_abs": float(diff.max()), "rel_l2": rel, "bit_equal": bool(np.array_equal(got, want_logits)),
                                  "greedy_ids_equal": bool(np.array_equal(got_all, want_picks)), "tolerance": {"max_abs": 2e-2, "rel_l2": 1e-3}}
            except Exception as e:  # the baseline is reported, never required
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"failed: {e}"}
        if tp_line is not None:
            line["tensor_parallel"] = tp_line
        print(json.dumps(line), flush=True)
    sess.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
