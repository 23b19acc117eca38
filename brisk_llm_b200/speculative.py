"""Lookup-draft speculative decoding over an Engine-shaped session: the caller of the token loop for the
batch-verify workload. Mirrors brisk-llm's LookupDrafter and Speculator (src/speculative.cpp:45-118) so the same
loop can run over CudaSession; the session only sees eval / eval_all / rollback / position.
"""
from __future__ import annotations

import numpy as np

MAX_NGRAM = 3
MAX_BACKOFF = 32


class LookupDrafter:
    """Guesses by finding the most recent earlier occurrence of the last 3, 2 or 1 tokens and copying what followed."""

    def __init__(self):
        self.history: list[int] = []

    def observe(self, tokens) -> None:
        self.history.extend(int(t) for t in tokens)

    def draft(self, count: int) -> list[int]:
        h, n = self.history, len(self.history)
        for ngram in range(min(MAX_NGRAM, n), 0, -1):
            suffix = h[n - ngram:]
            for start in range(n - ngram - 1, -1, -1):
                if h[start:start + ngram] == suffix:
                    begin = start + ngram
                    return h[begin:begin + min(count, n - begin)]
        return []


class Speculator:
    def __init__(self, target, drafter, carry: int, draft_tokens: int):
        self.target, self.drafter, self.carry = target, drafter, int(carry)
        self.draft_tokens = min(draft_tokens, 63)
        self.backoff = self.last_backoff = 0
        self.stats = {"rounds": 0, "plain": 0, "drafted": 0, "accepted": 0}

    def step(self) -> list[int]:
        if self.backoff > 0:
            self.backoff -= 1
            nxt = int(np.argmax(self.target.eval([self.carry])))
            self.drafter.observe([nxt])
            self.carry = nxt
            self.stats["plain"] += 1
            return [nxt]
        guesses = self.drafter.draft(self.draft_tokens)
        base = self.target.position()
        logits = self.target.eval_all([self.carry] + guesses)
        settled, accepted = [], 0
        nxt = int(np.argmax(logits[0]))
        while accepted < len(guesses) and guesses[accepted] == nxt:
            settled.append(nxt)
            accepted += 1
            nxt = int(np.argmax(logits[accepted]))
        settled.append(nxt)
        self.target.rollback(base + 1 + accepted)
        self.drafter.observe(settled)
        self.carry = nxt
        self.stats["rounds"] += 1
        self.stats["drafted"] += len(guesses)
        self.stats["accepted"] += accepted
        if accepted == 0 and guesses:
            self.last_backoff = min(MAX_BACKOFF, 1 if self.last_backoff == 0 else self.last_backoff * 2)
            self.backoff = self.last_backoff
        else:
            self.last_backoff //= 2
        return settled


def speculate(session, prompt, draft_tokens: int, want: int):
    """Evaluates prompt[:-1], then runs rounds until `want` tokens are settled. Returns (tokens, stats)."""
    prompt = [int(t) for t in prompt]
    drafter = LookupDrafter()
    drafter.observe(prompt)
    if len(prompt) > 1:
        session.eval(prompt[:-1])
    spec = Speculator(session, drafter, prompt[-1], draft_tokens)
    out: list[int] = []
    while len(out) < want:
        out.extend(spec.step())
    return np.array(out[:want], np.int32), spec.stats
