"""A request's numbers: how many tokens went in and came out, and when.

The reference fills such a record inside its generation loop and defines the decode rate
without the first token, which belongs to the time to first token
(src/mlx_omnia/engine/generate.py:260-357). Here the generation loop stamps the clock where it
already learns of a token (when a step's chosen ids have arrived on the host), so measuring
costs no synchronisation of its own.
"""

from __future__ import annotations

import time
from dataclasses import dataclass


@dataclass
class Meter:
    prompt_tokens: int = 0
    completion_tokens: int = 0
    preemptions: int = 0
    started: float | None = None  # the request was handed to the engine
    first_token: float | None = None
    last_token: float | None = None

    def begin(self, prompt_tokens: int) -> None:
        self.prompt_tokens = prompt_tokens
        self.started = time.perf_counter()

    def token(self) -> None:
        now = time.perf_counter()
        self.completion_tokens += 1
        if self.first_token is None:
            self.first_token = now
        self.last_token = now

    @property
    def ttft(self) -> float | None:
        """Seconds from the request's arrival to its first token (queueing, the prompt, one draw)."""
        if self.started is None or self.first_token is None:
            return None
        return self.first_token - self.started

    @property
    def decode_seconds(self) -> float | None:
        if self.first_token is None or self.last_token is None:
            return None
        return self.last_token - self.first_token

    @property
    def tokens_per_second(self) -> float | None:
        """Decoding only: the tokens after the first, over the time after the first."""
        elapsed = self.decode_seconds
        if elapsed is None or elapsed <= 0 or self.completion_tokens < 2:
            return None
        return (self.completion_tokens - 1) / elapsed

    def line(self) -> str:
        rate = self.tokens_per_second
        ttft = self.ttft
        return (f"prompt {self.prompt_tokens} tokens, completion {self.completion_tokens} tokens, "
                f"first token after {'-' if ttft is None else f'{ttft * 1e3:.1f} ms'}, "
                f"decode {'-' if rate is None else f'{rate:.1f} tokens/s'}"
                + (f", preempted {self.preemptions}x" if self.preemptions else ""))
