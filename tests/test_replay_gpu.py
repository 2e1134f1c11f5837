"""bin/trace_run, driven as a user drives it: a model folder, steps on standard input,
logits files out. The same requests are replayed whole, with the last 32 tokens one
by one, and in batches of unequal lengths that follow one another so that slots are
used again; in 32-bit and in bfloat16; all compared with the plain implementation."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import TINY, assert_close, plain_logits, prompts_for, tiny_config

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


class Trace:
    """Builds the steps of a schedule and remembers which (request, position) each
    output row of each step holds."""

    def __init__(self):
        self.steps, self.rows = [], {}

    def add(self, entries, end=()):
        n = len(self.steps)
        self.steps.append({"step": n, "entries": [{"id": rid, "tokens": toks, "want": want} for rid, toks, want, _ in entries],
                           "end": list(end)})
        self.rows[n] = [(rid, first + w) for rid, toks, want, first in entries for w in want]

    def batch(self, requests, prompt_lens):
        """requests: id -> tokens. All start together, then go on by single tokens; each
        ends when its tokens are used up."""
        fed = dict(zip(requests, prompt_lens))
        first = [(rid, requests[rid][:fed[rid]], list(range(fed[rid])), 0) for rid in requests]
        self.add(first, [rid for rid in requests if fed[rid] == len(requests[rid])])
        live = [rid for rid in requests if fed[rid] < len(requests[rid])]
        while live:
            entries = [(rid, [requests[rid][fed[rid]]], [0], fed[rid]) for rid in live]
            for rid in live:
                fed[rid] += 1
            ending = [rid for rid in live if fed[rid] == len(requests[rid])]
            self.add(entries, ending)
            live = [rid for rid in live if rid not in ending]


def run_trace(folder, dtype, trace, out_dir, max_tokens, vocab):
    text = "".join(json.dumps(s) + "\n" for s in trace.steps)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", str(max_tokens)],
                          input=text, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert done == [f"done {s['step']}" for s in trace.steps]
    got = {}
    for n, rows in trace.rows.items():
        path = Path(out_dir) / f"{n}.f32"
        if not rows:
            assert not path.exists()
            continue
        data = np.fromfile(path, dtype="<f4").reshape(len(rows), vocab)
        for row, key in zip(data, rows):
            got.setdefault(key, []).append(torch.from_numpy(row.copy()))
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", TINY)
def test_replay_schedules_against_plain(folders, name, dtype, tmp_path):
    vocab = tiny_config(name).vocab_size
    seqs = prompts_for(name, [40, 100, 71, 33, 150], seed=31)
    reqs = {f"r{i}": s for i, s in enumerate(seqs)}
    trace = Trace()
    # (1) each request alone and whole
    for rid, toks in reqs.items():
        trace.batch({rid + "w": toks}, [len(toks)])
    # (2) alone, the last 32 tokens one by one
    for rid, toks in reqs.items():
        trace.batch({rid + "d": toks}, [len(toks) - 32])
    # (3) batches of unequal lengths, one after another: slots and pages are used again
    trace.batch({"r0b": seqs[0], "r1b": seqs[1], "r2b": seqs[2]}, [8, 64, 70])
    trace.batch({"r3b": seqs[3], "r4b": seqs[4], "r0c": seqs[0]}, [1, 129, 39])
    # a step that wants nothing still fills the cache
    trace.add([("quiet", seqs[2][:50], [], 0)])
    trace.add([("quiet", seqs[2][50:], list(range(21)), 50)], ["quiet"])
    # the most that is live at once: three requests of the batches, each rounded up to 64
    max_tokens = 64 * (3 + 2 + 3)
    got = run_trace(folders[name], dtype, trace, tmp_path / "out", max_tokens, vocab)
    for key, rows in got.items():
        rid, pos = key
        seq = seqs[int(rid[1])] if rid != "quiet" else seqs[2]
        ref = plain_logits(folders[name], name, seq, dtype)[pos]
        for row in rows:
            assert_close(row[None], ref[None], dtype, f"{name} {dtype} request {rid} position {pos}")
    # every position of every schedule was produced
    for i, s in enumerate(seqs):
        for suffix in ("w", "d"):
            assert all((f"r{i}{suffix}", p) in got for p in range(len(s)))
    if dtype == "float32":  # the 32-bit path: the same logits however the tokens were cut or batched
        for i, s in enumerate(seqs):
            for p in range(len(s)):
                whole = got[(f"r{i}w", p)][0]
                assert torch.equal(whole, got[(f"r{i}d", p)][0])
                other = got.get((f"r{i}b", p))
                if other:
                    assert torch.equal(whole, other[0])


def test_replay_refuses_a_trace_that_does_not_fit(folders, tmp_path):
    seq = prompts_for("tiny_a", [200], seed=32)[0]
    text = json.dumps({"step": 0, "entries": [{"id": "a", "tokens": seq, "want": [0]}], "end": []}) + "\n"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folders["tiny_a"]), "--dtype",
                           "float32", "--out", str(tmp_path / "o"), "--max-tokens", "128"],
                          input=text, capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0 and "128" in proc.stderr
