"""Trace replay through ``bin/trace_run`` against the plain implementation: each request
whole; most of it in one step and the last 32 tokens one by one; portions of changing size
down to two tokens; and mixed, up to four live requests with so few pages that they are
used again.  In float32 and in bfloat16, for three tiny configurations."""
import os
import random

import numpy as np
import pytest
import torch

from helpers import TINY, TOL, TraceSession, make_model_folder, plain_logits, random_ids, rel_err, round64

pytestmark = pytest.mark.gpu

LENGTHS = {"tiny_a": [70, 150, 33, 200, 97, 260], "tiny_b": [45, 130, 64, 210, 31, 99],
           "tiny_c": [90, 300, 40, 170, 65, 230], "tiny_d": [120, 290, 36, 180, 75, 250]}
PORTIONS = [7, 2, 16, 3, 2, 33, 5, 2, 64, 11, 2, 17]


def _requests(name):
    vocab = TINY[name]["config"]["vocab_size"]
    return {f"r{i}": random_ids(n, vocab, seed=100 * i + len(name)) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module", params=[(n, d) for n in TINY for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def session(request, tmp_path_factory):
    name, dtype = request.param
    folder = str(tmp_path_factory.mktemp(f"model_{name}"))
    make_model_folder(folder, name)
    out = str(tmp_path_factory.mktemp(f"out_{name}_{dtype}"))
    reqs = _requests(name)
    # the mixed trace holds at most four requests: size the pool for the four longest, no more
    max_tokens = sum(sorted((round64(len(v)) for v in reqs.values()), reverse=True)[:4])
    s = TraceSession(folder, dtype, out, max_tokens, TINY[name]["block_size"], TINY[name]["config"]["vocab_size"])
    s.name, s.dtype, s.folder, s.requests = name, dtype, folder, reqs
    s.collected = {}
    yield s
    assert s.close() == 0


def _check(session, rid, positions, got, label):
    want = plain_logits(session.folder, session.requests[rid])[positions]
    err = rel_err(torch.from_numpy(np.ascontiguousarray(got)), want)
    assert err <= TOL[session.dtype], f"{label}: request {rid}, first bad position " \
        f"{_first_bad(got, want, positions, TOL[session.dtype])}, error {err:.3g}"
    session.collected.setdefault(label, {})[rid] = (list(positions), np.array(got))


def _first_bad(got, want, positions, tol):
    scale = float(want.abs().max())
    for i, p in enumerate(positions):
        if float((torch.from_numpy(np.ascontiguousarray(got[i])) - want[i]).abs().max()) > tol * scale:
            return p
    return None


def test_whole(session):
    for rid, ids in session.requests.items():
        got = session.step([{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], end=[rid])
        _check(session, rid, list(range(len(ids))), got, "whole")


def test_tail_one_by_one(session):
    for rid, ids in session.requests.items():
        head = max(1, len(ids) - 32)
        got = [session.step([{"id": rid, "tokens": ids[:head], "want": list(range(head))}])]
        for p in range(head, len(ids)):
            got.append(session.step([{"id": rid, "tokens": [ids[p]], "want": [0]}],
                                    end=[rid] if p == len(ids) - 1 else []))
        _check(session, rid, list(range(len(ids))), np.concatenate(got), "tail")


def test_portions(session):
    for k, (rid, ids) in enumerate(session.requests.items()):
        got, p, j = [], 0, k
        while p < len(ids):
            n = min(PORTIONS[j % len(PORTIONS)], len(ids) - p)
            j += 1
            got.append(session.step([{"id": rid, "tokens": ids[p:p + n], "want": list(range(n))}],
                                    end=[rid] if p + n == len(ids) else []))
            p += n
        _check(session, rid, list(range(len(ids))), np.concatenate(got), "portions")


def test_mixed(session):
    """Up to four live requests; portions of some beside single tokens of others; requests end and
    their pages go to the ones that start later (the pool holds four requests, six run)."""
    rng = random.Random(7)
    pending = list(session.requests.items())
    live = {}            # rid -> next position
    got = {rid: [] for rid, _ in pending}
    steps = 0
    while pending or live:
        while pending and len(live) < 4:
            rid, _ = pending.pop(0)
            live[rid] = 0
        entries, ending = [], []
        for rid in list(live):
            ids = session.requests[rid]
            p = live[rid]
            if rng.random() < 0.15 and len(live) > 1:
                continue                                    # left out of this step, goes on later
            tail = len(ids) - 24
            n = 1 if p >= tail else min(rng.choice([2, 3, 5, 9, 17, 30]), tail - p)
            entries.append({"id": rid, "tokens": ids[p:p + n], "want": list(range(n))})
            live[rid] = p + n
            if p + n == len(ids):
                ending.append(rid)
        if not entries:
            continue
        out = session.step(entries, end=ending)
        row = 0
        for e in entries:
            n = len(e["tokens"])
            got[e["id"]].append(out[row:row + n])
            row += n
        for rid in ending:
            del live[rid]
        steps += 1
    assert steps > 20
    for rid, ids in session.requests.items():
        _check(session, rid, list(range(len(ids))), np.concatenate(got[rid]), "mixed")


def test_cuts_agree(session):
    """The logits at a position do not depend on how the request was cut.  In float32 every sum of the
    path has an order that depends only on the token's position (products: one chain of K multiply-adds;
    norms: the block size follows the width; attention: key tiles aligned at multiples of 32 from key 0),
    so the four ways of cutting must agree to the bit.  In bfloat16 the kernels differ with the number of
    rows (weight streaming, tcgen05, the library) and the bound is a rounding of the activations."""
    for label, fn in (("whole", test_whole), ("tail", test_tail_one_by_one), ("portions", test_portions),
                      ("mixed", test_mixed)):
        if label not in session.collected:
            fn(session)                                     # run alone: make what is compared
    for label in ("tail", "portions", "mixed"):
        for rid, (_, ref) in session.collected["whole"].items():
            other = session.collected[label][rid][1]
            if session.dtype == "float32":
                same = np.array_equal(other, ref)
                where = None if same else int(np.argwhere((other != ref).any(axis=1))[0, 0])
                assert same, f"{label} against whole, request {rid}: first position that differs {where}, " \
                    f"largest difference {float(np.abs(other - ref).max()):.3g}"
            else:
                err = rel_err(torch.from_numpy(other), torch.from_numpy(ref))
                assert err <= 1.5e-2, f"{label} against whole, request {rid}: {err:.3g}"


def test_nothing_wanted_writes_no_file(session):
    ids = session.requests["r0"][:20]
    assert session.step([{"id": "nw", "tokens": ids[:10], "want": []}]) is None
    got = session.step([{"id": "nw", "tokens": ids[10:], "want": [9]}], end=["nw"])
    want = plain_logits(session.folder, session.requests["r0"])[19:20]
    assert rel_err(torch.from_numpy(got), want) <= TOL[session.dtype]
