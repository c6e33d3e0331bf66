"""Device-side token history: the matrix handed to the penalty / watermark stages must equal the zero-padded
matrix built from the host lists, through appends, departures, arrivals and batch merges."""
import random

import numpy as np
import torch

from tgi_b200.utils.history import TokenHistory


def naive(ids):
    L = max(len(x) for x in ids)
    out = np.zeros((len(ids), L), dtype=np.int64)
    for r, x in enumerate(ids):
        out[r, :len(x)] = x
    return torch.from_numpy(out)


def test_history_tracks_host_lists_through_batch_surgery():
    rng = random.Random(0)
    hist = TokenHistory("cpu", rows=2, capacity=4)
    live = {}
    next_id = 0
    for step in range(200):
        # arrivals
        for _ in range(rng.randint(0, 2)):
            live[next_id] = [rng.randint(1, 999) for _ in range(rng.randint(1, 40))]
            next_id += 1
        if not live:
            continue
        # departures
        for rid in [r for r in live if rng.random() < 0.05]:
            if len(live) > 1:
                del live[rid]
        # a step samples a subset of the batch, in any order
        active = rng.sample(sorted(live), rng.randint(1, len(live)))
        hist.retain(live.keys())
        got = hist.sync(active, [live[r] for r in active])
        assert torch.equal(got, naive([live[r] for r in active])), step
        # every sampled row grows by 1..3 ids (speculation accepts several); lists are append-only
        for r in active:
            live[r].extend(rng.randint(1, 999) for _ in range(rng.randint(1, 3)))
    assert set(hist.row_of) <= set(live)
    assert len(hist.free) + len(hist.row_of) == hist.buf.shape[0]


def test_history_uploads_only_new_ids(monkeypatch):
    hist = TokenHistory("cpu")
    a, b = list(range(1, 1001)), list(range(5, 505))
    hist.sync([7, 9], [a, b])
    seen = []
    real = torch.from_numpy

    def spy(arr):
        seen.append(arr.shape)
        return real(arr)

    monkeypatch.setattr(torch, "from_numpy", spy)
    a.append(4242)
    b.append(4343)
    out = hist.sync([7, 9], [a, b])
    assert seen == [(3, 2)]                      # two (row, position, token) triples, not 1501 ids
    assert out[0, 1000] == 4242 and out[1, 500] == 4343 and out[1, 501] == 0
