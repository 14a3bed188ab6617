"""bin/trace_run as a user runs it: a subprocess fed JSON steps on standard input.  The same
requests are replayed whole, with the last 32 tokens decoded one by one, and in batches
of unequal lengths whose shorter requests end earlier - in float32 and in bfloat16 - and
every logit row is compared with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import tiny_configs as tc
from helpers import assert_close, plain_logits

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build_trace(requests):
    """Steps for three modes over the same requests.  Returns (steps, expectation) where
    expectation[step] = list of (request index, [positions]) in output order."""
    steps, expect = [], {}

    def add(entries, end, rows):
        n = len(steps)
        steps.append({"step": n, "entries": entries, "end": end})
        if rows:
            expect[n] = rows

    # whole: each request alone, all positions wanted
    for r, tokens in enumerate(requests):
        add([{"id": f"w{r}", "tokens": tokens, "want": list(range(len(tokens)))}], [f"w{r}"],
            [(r, list(range(len(tokens))))])
    # last 32 one by one
    for r, tokens in enumerate(requests):
        head = max(len(tokens) - 32, 0)
        if head:
            add([{"id": f"l{r}", "tokens": tokens[:head], "want": list(range(head))}], [], [(r, list(range(head)))])
        for t in range(head, len(tokens)):
            add([{"id": f"l{r}", "tokens": [tokens[t]], "want": [0]}], [f"l{r}"] if t == len(tokens) - 1 else [],
                [(r, [t])])
    # batches of three that start together; prompts are about half of each request
    for begin in range(0, len(requests), 3):
        group = list(range(begin, min(begin + 3, len(requests))))
        fed = {r: max(1, len(requests[r]) // 2) for r in group}
        entries = [{"id": f"b{r}", "tokens": requests[r][:fed[r]], "want": [fed[r] - 1, 0] if fed[r] > 1 else [0]}
                   for r in group]
        add(entries, [f"b{r}" for r in group if fed[r] == len(requests[r])],
            [(r, [fed[r] - 1, 0] if fed[r] > 1 else [0]) for r in group])
        live = [r for r in group if fed[r] < len(requests[r])]
        while live:
            entries = [{"id": f"b{r}", "tokens": [requests[r][fed[r]]], "want": [0]} for r in live]
            rows = [(r, [fed[r]]) for r in live]
            for r in live:
                fed[r] += 1
            add(entries, [f"b{r}" for r in live if fed[r] == len(requests[r])], rows)
            live = [r for r in live if fed[r] < len(requests[r])]
    return steps, expect


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run(model_folders, tmp_path, name, dtype):
    folder = model_folders(name, dtype)
    top = tc.TINY[name]["max_position_embeddings"]
    lengths = [n for n in (7, 40, 1, 64, 100, 33) if n <= top]
    requests = [tc.random_tokens(name, n, 900 + i) for i, n in enumerate(lengths)]
    steps, expect = build_trace(requests)
    # most tokens live at once: a batch of three, each rounded up to 64
    budget = max(sum(-(-len(requests[r]) // 64) * 64 for r in range(b, min(b + 3, len(requests))))
                 for b in range(0, len(requests), 3))
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
         "--out", str(out), "--max-tokens", str(budget)],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    vocab = tc.TINY[name]["vocab_size"]
    refs = [plain_logits(folder, tokens, dtype) for tokens in requests]
    assert sorted(int(f[:-4]) for f in os.listdir(out)) == sorted(expect)
    for step, rows in expect.items():
        got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, vocab)
        want = np.concatenate([refs[r][positions] for r, positions in rows])
        assert_close(got, want, dtype, f"{name} {dtype} step {step}")


def test_trace_run_reports_a_full_cache(model_folders, tmp_path):
    folder = model_folders("A", "float32")
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1] * 60, "want": []},
                                     {"id": "b", "tokens": [2] * 10, "want": [9]}], "end": []}]
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
         "--out", str(tmp_path / "o"), "--max-tokens", "64"],
        input=json.dumps(steps[0]) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0 and "free" in proc.stderr


def random_trace(name, rng):
    """Batches of 1 to 20 requests that start together with unequal prompts and go on one token each, the
    shorter ones ending earlier; up to two batches live at once, their steps interleaved (a live request is not in
    every step); places wanted: none, the last, all, or a few in any order.  Returns (steps, expectation, requests,
    the most tokens held at once, each request's count rounded up to 64), expectation[step] = [(id, positions)]."""
    top, vocab = tc.TINY[name]["max_position_embeddings"], tc.TINY[name]["vocab_size"]
    steps, expect, requests, held, batches = [], {}, {}, {}, []
    peak, made, n_batches = 0, 0, int(rng.randint(2, 6))

    def add(entries, rows, end):
        nonlocal peak
        peak = max(peak, sum(-(-n // 64) * 64 for n in held.values()))
        steps.append({"step": len(steps), "entries": entries, "end": end})
        if rows:
            expect[len(steps) - 1] = rows
        for i in end:
            del held[i]

    while made < n_batches or batches:
        if made < n_batches and len(batches) < 2 and (not batches or rng.rand() < 0.3):
            ids = [f"r{made}_{i}" for i in range(int(rng.choice([1, 2, 3, 5, 8, 13, 20])))]
            fed, total = {}, {}
            entries, rows = [], []
            for i in ids:
                prompt = int(min(top - 2, rng.choice([1, 2, 7, 31, 63, 64, 65, 100, 129, 200])))
                total[i] = min(top, prompt + int(rng.choice([0, 1, 2, 5, 17, 40])))
                fed[i] = min(prompt, total[i])
                requests[i] = [int(t) for t in rng.randint(0, vocab, size=total[i])]
                kind = rng.randint(4)
                want = ([], [fed[i] - 1], list(range(fed[i])), [int(x) for x in rng.randint(0, fed[i], size=3)])[kind]
                entries.append({"id": i, "tokens": requests[i][:fed[i]], "want": want})
                if want:
                    rows.append((i, want))
                held[i] = fed[i]
            add(entries, rows, [i for i in ids if fed[i] == total[i]])
            alive = [i for i in ids if fed[i] < total[i]]
            if alive:
                batches.append({"ids": alive, "fed": fed, "total": total})
            made += 1
            continue
        batch = batches[int(rng.randint(len(batches)))]
        entries, rows = [], []
        for i in batch["ids"]:
            want = [0] if rng.rand() < 0.8 else []
            entries.append({"id": i, "tokens": [requests[i][batch["fed"][i]]], "want": want})
            if want:
                rows.append((i, [batch["fed"][i]]))
            batch["fed"][i] += 1
            held[i] = batch["fed"][i]
        end = [i for i in batch["ids"] if batch["fed"][i] == batch["total"][i]]
        add(entries, rows, end)
        batch["ids"] = [i for i in batch["ids"] if i not in end]
        if not batch["ids"]:
            batches.remove(batch)
    return steps, expect, requests, peak


@pytest.mark.parametrize("name,dtype,seed", [("D", "bfloat16", 4), ("B", "float32", 5), ("C", "bfloat16", 3), ("A", "float32", 1)])
def test_random_traces_with_the_cache_sized_to_the_token(model_folders, tmp_path, name, dtype, seed):
    """A trace drawn from a seed, the steps sent one at a time (the next only after `done <step>`), and
    --max-tokens exactly what the trace holds at its fullest."""
    folder = model_folders(name, dtype)
    steps, expect, requests, peak = random_trace(name, np.random.RandomState(seed))
    out = tmp_path / "out"
    proc = subprocess.Popen(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out),
         "--max-tokens", str(peak)], stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {s['step']}", (line, proc.stderr.read()[-2000:] if proc.poll() is not None else "")
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    vocab = tc.TINY[name]["vocab_size"]
    refs = {i: plain_logits(folder, tokens, dtype) for i, tokens in requests.items()}
    assert sorted(int(f[:-4]) for f in os.listdir(out)) == sorted(expect)   # a step that wants nothing writes nothing
    for step, rows in expect.items():
        got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, vocab)
        want = np.concatenate([refs[i][positions] for i, positions in rows])
        assert_close(got, want, dtype, f"{name} {dtype} seed {seed} step {step}")
