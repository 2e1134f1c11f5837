"""Token selection: greedy, and temperature sampling with counter-based draws.

The reference selects greedily only: ``argmax`` over the vocabulary, the lowest
index winning an exact tie (engine/engine.py:193,196 of
willzeng274/kernel-rush-kawk). Temperature sampling is this library's addition.
It uses the Gumbel-max form, token = argmax_i(logit_i / temperature + g_i) with
g_i = -log(-log(u_i)), which is a draw from softmax(logits / temperature) made in
one pass over the logits. The uniforms come from a 32-bit mixing hash of (seed,
request, step, i): u_i = ((hash >> 9) + 0.5) / 2^23. A request's draw therefore
depends on its own index and step only, never on what else is in its batch.
Both run in one CUDA kernel over float32 logits.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0


class Sampler:
    """Picks one token per row of ``logits`` on the device and brings them to the host."""

    def __init__(self, ops, device):
        self.ops = ops
        self.device = torch.device(device)
        self._pinned = None
        self._requests = None
        self._requests_host: list[int] = []

    def select(self, logits: torch.Tensor, params: SamplingParams, requests: list[int], step: int) -> list[int]:
        """logits [n, vocab] float32; requests: each row's request index; step: how many
        tokens each of these requests has generated before this one."""
        return self.finish(self.launch(logits, params, requests, step))

    def launch(self, logits: torch.Tensor, params: SamplingParams, requests: list[int], step: int):
        """Start the selection and the copy of its result to the host; ``finish`` waits for it."""
        n = logits.shape[0]
        if self._requests_host != list(requests):
            self._requests_host = list(requests)
            self._requests = torch.tensor(requests, dtype=torch.int32).to(self.device)
        tokens = self.ops.select_tokens(logits, float(params.temperature), int(params.seed), self._requests, int(step))
        if self._pinned is None or self._pinned.numel() < n + 1:
            self._pinned = torch.empty(max(n, 64) + 1, dtype=torch.int32, pin_memory=self.device.type == "cuda")
        host = self._pinned[:n + 1]
        host[:n].copy_(tokens, non_blocking=True)
        error = getattr(self.ops, "error", None)  # the kernels' error word rides along with the tokens
        if error is not None:
            host[n:].copy_(error, non_blocking=True)
        else:
            host[n] = 0
        return host

    def finish(self, host) -> list[int]:
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        row = host.tolist()
        if row[-1]:
            self.ops.check()  # raises with the flag's meaning and clears the word
        return row[:-1]
