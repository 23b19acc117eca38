"""Per-phase device time of the token loop on a seeded synthetic model (the counterpart of `BRISK_PROFILE=1 brisk
generate`, brisk-llm src/main.cpp:302-306): where a prefill and a decode step spend their time.

    python -m brisk_llm_b200.phases --config qwen3-0.6b-q4_0 [--prompt 512] [--context 2048] [--decode 16]

Uses brisk_cuda_profile: every phase is bracketed by CUDA events and the single-token step runs kernel by kernel, so
the totals are slower than the graph-replayed step (whose time is printed beside them); read the shares.
"""
from __future__ import annotations

import argparse
from dataclasses import replace

from . import engine, synth


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="qwen3-0.6b-q4_0", choices=sorted(synth.PRESETS))
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--decode", type=int, default=16)
    ap.add_argument("--verify", type=int, default=0, help="also break down an eval_all of this many tokens (a speculative verify step)")
    a = ap.parse_args()
    spec = replace(synth.PRESETS[a.config], context=a.context)
    model = synth.generate(spec, seed=0, share_layers=spec.layers * spec.hidden * spec.ffn > 1e9)
    ids = synth.random_tokens(spec, a.prompt, seed=1)
    with engine.CudaSession(model, max_context=a.context) as s:
        s.eval(ids)
        s.rollback(0)
        s.profile(True)
        s.eval(ids)
        p = s.profile(True)
        total = sum(v["ms"] for v in p.values())
        print(f"{a.config}: prefill of {a.prompt} tokens, {total:.2f} ms in phases")
        for k, v in p.items():
            if v["calls"]:
                print(f"  {k:10s} {v['ms']:9.3f} ms  {100 * v['ms'] / total:5.1f}%  ({v['calls']} calls)")
        s.generate_greedy(5, a.decode)
        p = s.profile(False)
        total = sum(v["ms"] for v in p.values())
        print(f"decode at context {a.prompt}..{a.prompt + a.decode}: {1000 * total / a.decode:.1f} us per token in phases (profiled, kernel by kernel)")
        for k, v in p.items():
            if v["calls"]:
                print(f"  {k:10s} {1000 * v['ms'] / a.decode:9.1f} us  {100 * v['ms'] / total:5.1f}%")
        s.generate_greedy(5, a.decode)
        print(f"  graph-replayed step, unprofiled: {1000 * s.stats()['device_ms'] / a.decode:.1f} us per token")
        if a.verify:
            pos = s.position()
            probe = synth.random_tokens(spec, a.verify, seed=3)
            s.eval_all(probe)
            s.rollback(pos)
            s.profile(True)
            s.eval_all(probe)
            p = s.profile(False)
            s.rollback(pos)
            total = sum(v["ms"] for v in p.values())
            print(f"eval_all of {a.verify} tokens at context {pos}: {1000 * total:.1f} us in phases")
            for k, v in p.items():
                if v["calls"]:
                    print(f"  {k:10s} {1000 * v['ms']:9.1f} us  {100 * v['ms'] / total:5.1f}%")
            s.eval_all(probe)
            print(f"  unprofiled: {1000 * s.stats()['device_ms']:.1f} us")


if __name__ == "__main__":
    main()
