"""The native layout of a step's batch (csrc/host_runtime.cpp, lmsf_cm_build_batch) against a restatement in Python,
on random batches: prompt portions beside single tokens, wanted places, windows whose pages have been given back,
tokens that are still on the device, fixed table widths and stand-in requests that fill a batch up to a graph size."""
import random

import numpy as np

from lmsf_b200.cache import native
from lmsf_b200.cache.manager import CacheManager, GroupSpec

Q_TILE = 64
NAMES = ["token_ids", "positions", "token_seq", "cu_q", "ctx_len", "state_slot", "patch_dst", "patch_src", "rows",
         "dec_ids", "tile_seq", "tile_q0", "tile128_seq", "tile128_q0"]


def build(mgr, entries, static_blocks, pad_to, null_pages):
    S, G = len(entries), len(mgr.groups)
    rids = np.asarray([mgr.native_id(e["id"]) for e in entries], dtype=np.int64)
    q = np.asarray([len(e["tokens"]) for e in entries], dtype=np.int32)
    tok = np.asarray([t for e in entries for t in e["tokens"]], dtype=np.int32)
    wc = np.asarray([len(e["want"]) for e in entries], dtype=np.int32)
    wf = np.asarray([w for e in entries for w in e["want"]] or [0], dtype=np.int32)
    lf = np.asarray([e["last_from"] for e in entries], dtype=np.int32)
    seg, info = np.zeros(2 * (14 + G), dtype=np.int32), np.zeros(7 + G, dtype=np.int32)
    ctx = np.zeros(max(S, pad_to), dtype=np.int32)
    nul = np.asarray(null_pages, dtype=np.int32)
    p = lambda a: a.ctypes.data
    lib = native.lib()
    args = (mgr.handle(), S, p(rids), p(q), p(tok), p(wc), p(wf), p(lf), static_blocks, Q_TILE, pad_to, p(nul))
    assert lib.lmsf_cm_build_batch(*args, None, 0, p(seg), p(info), p(ctx)) == 0
    out = np.full(int(info[6]), 12345, dtype=np.int32)
    if info[6] > 4:
        assert lib.lmsf_cm_build_batch(*args, p(out), int(info[6]) - 1, p(seg), p(info), p(ctx)) == -4     # too small a buffer
    assert lib.lmsf_cm_build_batch(*args, p(out), out.size, p(seg), p(info), p(ctx)) == 0
    names = NAMES + [f"bt{g}" for g in range(G)]
    view = {n: out[seg[2 * i]:seg[2 * i] + seg[2 * i + 1]] for i, n in enumerate(names)}
    assert all(int(seg[2 * i]) % 4 == 0 for i in range(len(names))), "segments start on 16-byte boundaries"
    return view, info, ctx


def check_batch(rng, window):
    bs = rng.choice([1, 4, 16])
    groups = [GroupSpec(None)] + ([GroupSpec(window)] if window else [])
    mgr = CacheManager(groups, [4000] * len(groups), bs, 16)
    entries, cached = [], {}
    for i in range(rng.randint(1, 9)):
        rid = f"r{i}"
        mgr.add(rid)
        n0 = rng.choice([0, 0, 3, 50, 130])             # tokens that earlier steps left in the cache
        if n0:
            mgr.reserve(rid, n0)
            mgr.commit(rid, n0)
        n = rng.choice([1, 1, 1, 2, 7, 64, 65, 200])
        mgr.reserve(rid, n)
        cached[rid] = n0
        want = sorted(rng.sample(range(n), rng.randint(0, min(n, 3))))
        entries.append(dict(id=rid, tokens=[rng.randrange(1000) for _ in range(n)], want=want,
                            last_from=rng.randrange(8) if rng.random() < 0.2 else -1))
    S = len(entries)
    decode_only = all(len(e["tokens"]) == 1 for e in entries)
    pad_to = rng.choice([0, S + 3]) if decode_only else 0
    widest = max(len(mgr.block_table(e["id"], g)) for e in entries for g in range(len(groups)))
    static_blocks = rng.choice([0, widest + 5])
    null_pages = [4000 + g for g in range(len(groups))]
    v, info, ctx = build(mgr, entries, static_blocks, pad_to, null_pages)

    S_pad = max(S, pad_to)
    q = [len(e["tokens"]) for e in entries] + [1] * (S_pad - S)
    N = sum(q)
    assert info[0] == N and len(v["token_ids"]) == N
    tokens = [t for e in entries for t in e["tokens"]] + [0] * (S_pad - S)
    assert v["token_ids"].tolist() == tokens
    cu = np.concatenate([[0], np.cumsum(q)]).tolist()
    assert v["cu_q"].tolist() == cu
    starts = [cached[e["id"]] for e in entries] + [0] * (S_pad - S)
    assert v["positions"].tolist() == [starts[s] + j for s in range(S_pad) for j in range(q[s])]
    assert v["token_seq"].tolist() == [s for s in range(S_pad) for _ in range(q[s])]
    assert v["ctx_len"].tolist() == [starts[s] + q[s] for s in range(S_pad)] == ctx[:S_pad].tolist()
    assert v["state_slot"].tolist() == [mgr.state_slot(e["id"]) for e in entries] + [mgr.num_state_slots] * (S_pad - S)
    assert v["patch_dst"].tolist() == [cu[s + 1] - 1 if e["last_from"] >= 0 else -1 for s, e in enumerate(entries)] + [-1] * (S_pad - S)
    assert v["patch_src"].tolist() == [max(e["last_from"], 0) for e in entries] + [0] * (S_pad - S)
    assert info[5] == int(any(e["last_from"] >= 0 for e in entries))
    rows = [cu[s] + w for s, e in enumerate(entries) for w in e["want"]] + [cu[s] for s in range(S, S_pad)]
    assert v["rows"].tolist() == rows and info[1] == len(rows)
    assert v["dec_ids"].tolist() == [s for s in range(S_pad) if q[s] == 1] and info[2] == len(v["dec_ids"])
    for tile, seq_name, q0_name, count in ((Q_TILE, "tile_seq", "tile_q0", info[3]), (2 * Q_TILE, "tile128_seq", "tile128_q0", info[4])):
        got = list(zip(v[seq_name].tolist(), v[q0_name].tolist()))
        want = [(s, q0) for s in range(S) if q[s] > 1 for q0 in range(0, q[s], tile)]
        assert sorted(got) == sorted(want) and count == len(want)
        keys = [starts[s] + min(q0 + tile, q[s]) for s, q0 in got]          # the keys a tile sees: most first
        assert keys == sorted(keys, reverse=True)
    for g in range(len(groups)):
        width = int(info[7 + g])
        assert width >= max(static_blocks, 1) and (static_blocks == 0 or width == static_blocks)
        bt = v[f"bt{g}"].reshape(S_pad, width)
        for s, e in enumerate(entries):
            table = mgr.block_table(e["id"], g)
            assert bt[s, :len(table)].tolist() == table and (bt[s, len(table):] == -1).all()
        for s in range(S, S_pad):
            assert bt[s, 0] == null_pages[g] and (bt[s, 1:] == -1).all()
    if window:      # a window that has passed gives pages back: those entries read -1
        for e in entries:
            mgr.commit(e["id"], len(e["tokens"]))
        long_ones = [e for e in entries if cached[e["id"]] + len(e["tokens"]) > window + 2 * bs]
        for e in long_ones:
            assert mgr.block_table(e["id"], 1)[0] == -1 and mgr.block_table(e["id"], 0)[0] >= 0
    mgr.check_invariants()


def test_native_layout_on_random_batches():
    rng = random.Random(0)
    for i in range(300):
        check_batch(rng, window=rng.choice([None, None, 8, 40]))


def test_unknown_request_is_refused():
    mgr = CacheManager([GroupSpec(None)], [8], 4, 4)
    mgr.add("a")
    z = np.zeros(8, dtype=np.int32)
    one = np.ones(1, dtype=np.int32)
    rid = np.asarray([987654], dtype=np.int64)
    p = lambda a: a.ctypes.data
    seg, info = np.zeros(30, dtype=np.int32), np.zeros(8, dtype=np.int32)
    rc = native.lib().lmsf_cm_build_batch(mgr.handle(), 1, p(rid), p(one), p(z), p(z), p(z), p(z), 0, Q_TILE, 0, p(z), None, 0,
                                          p(seg), p(info), p(z))
    assert rc == -2
