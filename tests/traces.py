"""Builders of replay traces (the JSON steps that bin/trace_run reads) and two ways of running them:
inside the test process through the engine's step function, or through the program itself."""
import json
import os
import random
import subprocess
import sys
import tempfile

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def whole(requests, tail=0):
    """Each request alone: all but the last `tail` tokens in one step, the rest one by one."""
    steps, k = [], 0
    for rid, toks in requests.items():
        head = len(toks) - tail
        if head > 0:
            steps.append({"step": k, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
            k += 1
        for i in range(max(head, 0), len(toks)):
            steps.append({"step": k, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}], "end": []})
            k += 1
        steps[-1]["end"] = [rid]
    return steps


def portions(requests, sizes):
    """Each request alone, cut into portions of changing size (cycled)."""
    steps, k = [], 0
    for rid, toks in requests.items():
        i, j = 0, 0
        while i < len(toks):
            n = min(sizes[j % len(sizes)], len(toks) - i)
            steps.append({"step": k, "entries": [{"id": rid, "tokens": toks[i:i + n], "want": list(range(n))}], "end": []})
            i, j, k = i + n, j + 1, k + 1
        steps[-1]["end"] = [rid]
    return steps


def mixed(requests, seed, max_live=4, sizes=(7, 2, 13, 3, 29, 2, 5), tail=12):
    """Up to `max_live` requests at a time: portions of some beside single tokens of others; a request may
    sit a step out; finished requests end and the next one starts, so their pages are used again."""
    rng = random.Random(seed)
    pending = list(requests.items())
    live = {}          # rid -> [tokens, done, portion counter]
    steps, k = [], 0
    while pending or live:
        while pending and len(live) < max_live:
            rid, toks = pending.pop(0)
            live[rid] = [toks, 0, rng.randrange(len(sizes))]
        chosen = [rid for rid in live if rng.random() < 0.7] or [rng.choice(list(live))]
        entries, end = [], []
        for rid in chosen:
            toks, done, j = live[rid]
            left = len(toks) - done
            n = 1 if left <= tail else min(sizes[j % len(sizes)], left - tail)
            entries.append({"id": rid, "tokens": toks[done:done + n], "want": list(range(n))})
            live[rid][1] += n
            live[rid][2] += 1
            if live[rid][1] == len(toks):
                end.append(rid)
        rng.shuffle(entries)
        for rid in end:
            del live[rid]
        steps.append({"step": k, "entries": entries, "end": end})
        k += 1
    return steps


def many_live(requests, tail, per_step=8):
    """All requests live at once: their prompts (all but the last `tail` tokens) arrive `per_step` requests a step,
    the newcomers' portions beside single tokens of those that are already decoding; then every step brings one
    token of every request until all are through."""
    rids = list(requests)
    done = {r: 0 for r in rids}
    steps, k, started = [], 0, 0
    while any(done[r] < len(requests[r]) for r in rids):
        entries, end = [], []
        for r in rids[:started]:
            if done[r] < len(requests[r]):
                entries.append({"id": r, "tokens": [requests[r][done[r]]], "want": [0]})
                done[r] += 1
        for r in rids[started:started + per_step]:
            head = max(1, len(requests[r]) - tail)
            entries.append({"id": r, "tokens": requests[r][:head], "want": [head - 1]})
            done[r] = head
        started = min(len(rids), started + per_step)
        steps.append({"step": k, "entries": entries, "end": []})
        k += 1
    steps[-1]["end"] = rids
    return steps


def dropped_and_replayed(requests, victim, cut, sizes=(9, 2, 17, 5)):
    """Portions of all requests in turn; `victim` is ended after `cut` of its tokens (what it holds is given back,
    as when a scheduler preempts it) while the others go on, and later starts again from its first token."""
    steps, k = [], 0
    done = {r: 0 for r in requests}
    dropped = False
    j = 0
    while any(done[r] < len(requests[r]) for r in requests):
        entries, end = [], []
        for r, toks in requests.items():
            if done[r] >= len(toks):
                continue
            n = min(sizes[j % len(sizes)], len(toks) - done[r])
            j += 1
            if r == victim and not dropped and done[r] + n >= cut:
                n = max(1, cut - done[r])
            entries.append({"id": r, "tokens": toks[done[r]:done[r] + n], "want": list(range(n))})
            done[r] += n
            if r == victim and not dropped and done[r] >= cut:
                end.append(r)                  # freed in the middle of its prompt ...
                done[r] = 0                    # ... and replayed from token 0 in the steps that follow
                dropped = True
            elif done[r] == len(toks):
                end.append(r)
        steps.append({"step": k, "entries": entries, "end": end})
        k += 1
    return steps


def max_live_tokens(steps, round_to=64):
    """The --max-tokens a trace needs: most tokens held at any time, each request rounded up."""
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum((n + round_to - 1) // round_to * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def collect(steps, outputs):
    """{(request, position): logits row} from per-step outputs {step: array [wanted, vocab]}."""
    pos, rows = {}, {}
    for s in steps:
        out = outputs.get(s["step"])
        r = 0
        for e in s["entries"]:
            p0 = pos.get(e["id"], 0)
            for w in e["want"]:
                rows[(e["id"], p0 + w)] = out[r]
                r += 1
            pos[e["id"]] = p0 + len(e["tokens"])
        for rid in s["end"]:
            pos.pop(rid, None)
        assert out is None or r == out.shape[0]
    return rows


_runners = {}


def run_inprocess(folder, dtype, steps, block_size, max_tokens, max_live=8):
    """Drives ModelRunner + CacheManager exactly as bin/trace_run does."""
    from lmsf_b200.engine.factory import build_model
    from lmsf_b200.engine.model_runner import ModelRunner, StepEntry
    dev = torch.device("cuda:0")
    key = (folder, dtype)
    if key not in _runners:
        _runners[key] = build_model(folder, dtype, dev)
    model, _, tdt = _runners[key]
    pages = max(1, (max_tokens + block_size - 1) // block_size)
    runner = ModelRunner(model, tdt, dev, block_size, num_blocks=pages, max_num_seqs=max_live)
    mgr = runner.make_cache_manager()
    outputs = {}
    for s in steps:
        entries = []
        for e in s["entries"]:
            if not mgr.has(e["id"]):
                mgr.add(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        if entries:
            lg = runner.step(entries, mgr)
            if lg.shape[0]:
                outputs[s["step"]] = lg.float().cpu().numpy()
        for rid in s["end"]:
            mgr.free(rid)
        mgr.check_invariants()
    assert all(p.num_free == p.num_blocks for p in mgr.pools)
    return outputs


def run_program(folder, dtype, steps, max_tokens, env=None):
    """Runs bin/trace_run as a user would and reads back what it wrote."""
    out = tempfile.mkdtemp(prefix="lmsf_trace_")
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out,
           "--max-tokens", str(max_tokens)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    for s in steps:                                  # the next step only after "done <step>"
        proc.stdin.write(json.dumps(s) + "\n")
        proc.stdin.flush()
        line = proc.stdout.readline().strip()
        assert line == f"done {s['step']}", line
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0
    vocab = json.load(open(os.path.join(folder, "config.json")))["vocab_size"]
    outputs = {}
    for s in steps:
        p = os.path.join(out, f"{s['step']}.f32")
        n = sum(len(e["want"]) for e in s["entries"])
        assert os.path.exists(p) == (n > 0)
        if n:
            outputs[s["step"]] = np.fromfile(p, dtype="<f4").reshape(n, vocab)
    return outputs
