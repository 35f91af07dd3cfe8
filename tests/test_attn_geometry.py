"""Host model of the attention kernels' index logic (``csrc/attn_common.cuh`` and the work lists of
``csrc/attn_bwd_tcgen05.cu``): the per-row key intervals of the own-chunk patterns, the segment geometry, and the
(sequence, query tile) lists a key block walks.  The model restates the device functions line by line in Python and is
checked against the mask matrices of ``ops.attention``: every (query, key) pair the statement allows is met by exactly one
(key block, work item), with the mask the kernel would apply, and no pair outside it."""
import itertools

import pytest
import torch

from util import ROOT  # noqa: F401
from dttt_b200.ops import attention as A

FULL, CAUSAL, SPLIT, BLOCK, READ = range(5)
BK = 128


def row_mask(mode, param, i, Kn, Cq):
    own = Kn - Cq
    s2, e2 = 1, 0
    if mode == CAUSAL:
        e1 = own + i
    elif mode == SPLIT:
        e1 = own + max(i, param - 1)
    elif mode == BLOCK:
        e1 = own + (i // param + 1) * param - 1
    elif mode == READ:
        e1 = own - Cq + (i // param) * param - 1
        s2 = own + (i // param) * param
        e2 = min(s2 + param - 1, Kn - 1)
    else:
        e1 = Kn - 1
    return min(e1, Kn - 1), s2, e2


def parse(p):
    name, _, arg = p.partition(":")
    return {"full": FULL, "causal": CAUSAL, "split": SPLIT, "block": BLOCK, "read": READ}[name], int(arg) if arg else 0


@pytest.mark.parametrize("pattern", ["full", "causal", "split:5", "split:16", "block:4", "block:16", "read:4", "read:8"])
def test_row_intervals_equal_the_mask_matrices(pattern):
    C, lead = 16, 24
    mode, param = parse(pattern)
    own = A._own_part_mask(pattern, C, None)
    Kn = lead + (2 * C if mode == READ else C)
    for i in range(C):
        e1, s2, e2 = row_mask(mode, param, i, Kn, C)
        vis = [(j <= e1) or (s2 <= j <= e2) for j in range(Kn)]
        want = [True] * (Kn - (own.shape[1] if own is not None else 0)) + ([bool(x) for x in own[i]] if own is not None else [])
        assert vis == want, (pattern, i)


def seq_geom(sg, v, C):
    per_b = sg["streams"] * sg["chunks"]
    c, s = v % sg["chunks"], (v // sg["chunks"]) % sg["streams"]
    nv = min(sg["first"] + c, sg["W"])
    if sg["reach"] >= 0:
        nv = min(nv, sg["reach"])
    mode, param = sg["modes"][s]
    Kn1 = nv * C + (C if mode == READ else 0)
    return dict(Kn=Kn1 + C, Kn1=Kn1, mode=mode, param=param, kb=v // per_b, row0=(sg["W"] + c - nv) * C, nv=nv, stream=s, chunk=c)


def work_items(sg, C, z, jb, nqt):
    """The list CTA (jb, z) builds in the segment form: ``[(v, qt, needs_mask, kpos0)]``, or None when the CTA exits."""
    bb, st = z // sg["streams"], z % sg["streams"]
    second = st != 1
    klen = sg["chunks"] * C if second else (sg["W"] + sg["chunks"]) * C
    if jb * BK >= klen:
        return None
    krow = jb * BK
    per_b = sg["streams"] * sg["chunks"]
    out = []

    def consider(v, G, kpos0):
        for qt in range(nqt):
            i0, i1 = qt * BK, min(qt * BK + BK - 1, C - 1)
            a, zz = row_mask(G["mode"], G["param"], i0, G["Kn"], C), row_mask(G["mode"], G["param"], i1, G["Kn"], C)
            if not ((kpos0 <= zz[0]) or (kpos0 + BK - 1 >= a[1] and kpos0 <= zz[2])):
                continue
            whole = (kpos0 + BK - 1 <= a[0]) or (kpos0 >= zz[1] and kpos0 + BK - 1 <= a[2])
            out.append((v, qt, not (whole and kpos0 + BK <= G["Kn"]), kpos0))
    if second:
        c = krow // C
        v = bb * per_b + st * sg["chunks"] + c
        G = seq_geom(sg, v, C)
        consider(v, G, G["Kn"] - C + (krow - c * C))
    else:
        kc = krow // C - sg["W"]
        for c in range(max(kc, 0), min(kc + sg["W"] + 1, sg["chunks"])):
            for s2 in range(sg["streams"]):
                v = bb * per_b + s2 * sg["chunks"] + c
                G = seq_geom(sg, v, C)
                kpos0 = krow - G["row0"]
                reach_rows = G["nv"] * C + (C if (s2 == 1 or G["mode"] == READ) else 0)
                if 0 <= kpos0 < reach_rows:
                    consider(v, G, kpos0)
    return out


@pytest.mark.parametrize("streams,chunks,W,first,reach,patterns", [
    (3, 4, 2, 0, -1, ("full", "full", "causal")),
    (3, 3, 2, 5, -1, ("full", "full", "causal")),
    (2, 5, 3, 1, 2, ("full", "full")),
    (4, 2, 4, 0, -1, ("full", "block:64", "split:32", "causal")),
    (3, 2, 0, 0, -1, ("causal", "full", "full")),
])
def test_segment_work_lists_cover_every_visible_pair_once(streams, chunks, W, first, reach, patterns):
    C, B = 256, 2
    sg = dict(streams=streams, chunks=chunks, W=W, first=first, reach=reach, modes=[parse(p) for p in patterns])
    nqt = C // BK
    # the statement: per (b, s, c) which rows of the clean buffer / of its own keys a query row sees
    seen = {}
    for z, jb in itertools.product(range(B * streams), range((W + chunks) * C // BK)):
        items = work_items(sg, C, z, jb, nqt)
        if items is None:
            continue
        bb, st = z // streams, z % streams
        assert len(items) <= 512
        for v, qt, masked, kpos0 in items:
            G = seq_geom(sg, v, C)
            for i in range(qt * BK, qt * BK + BK):
                e1, s2, e2 = row_mask(G["mode"], G["param"], i, G["Kn"], C)
                for kr in range(BK):
                    kp = kpos0 + kr
                    vis = (kp <= e1) or (s2 <= kp <= e2)
                    if not masked:
                        assert vis
                    if vis:
                        key = (v, i, kp)
                        assert key not in seen, key
                        # which buffer row this key position is, as the forward reads it
                        seen[key] = ("own", st, jb * BK + kr) if st != 1 else ("clean", bb, jb * BK + kr)
    for v in range(B * streams * chunks):
        G = seq_geom(sg, v, C)
        own = A._own_part_mask(patterns[G["stream"]], C, None)
        for i in range(C):
            for kp in range(G["Kn"]):
                vis = True if kp < G["Kn"] - C or own is None else bool(own[i, kp - (G["Kn"] - C)])
                assert ((v, i, kp) in seen) == vis, (v, i, kp)
                if vis:
                    where = seen[(v, i, kp)]
                    if kp < G["Kn1"] or G["stream"] == 1:
                        assert where == ("clean", G["kb"], G["row0"] + kp), (v, i, kp, where)       # the clean buffer, in place
                    else:
                        assert where == ("own", G["stream"], G["chunk"] * C + kp - G["Kn1"]), (v, i, kp, where)
