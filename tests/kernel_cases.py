"""Shared builders of kernel test cases (imported by the kernel tests and by the tests of the
allocation-free entry point)."""

from __future__ import annotations

import math

import torch

from plain_qwen2 import plain_causal_attention

DEV = "cuda:0"


def paged_case(nh, nkv, D, page, q_lens, befores, dtype, seed, window=0):
    """Random requests laid out in a shuffled paged cache; returns device tensors and the plain result."""
    from tokenmill_b200.parts.attention_plan import tiles_for
    import numpy as np

    g = torch.Generator().manual_seed(seed)
    S = len(q_lens)
    G = nh // nkv
    totals = [b + n for b, n in zip(befores, q_lens)]
    n_pages = sum(-(-t // page) for t in totals) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    kc = torch.randn(n_pages, page, nkv, D, generator=g).to(dtype)     # stale noise in every unused slot
    vc = torch.randn(n_pages, page, nkv, D, generator=g).to(dtype)
    W = max(-(-t // page) for t in totals)
    table = torch.zeros(S, W, dtype=torch.int32)
    qs, refs = [], []
    for s in range(S):
        k = torch.randn(totals[s], nkv, D, generator=g).to(dtype)
        v = torch.randn(totals[s], nkv, D, generator=g).to(dtype)
        q = torch.randn(q_lens[s], nh, D, generator=g).to(dtype)
        if totals[s] > 40:                                           # one far key dominates one query head
            q[-1, 0] = 0
            q[-1, 0, 0] = 6.0
            k[3, 0] = 0
            k[3, 0, 0] = 6.0 * math.sqrt(D) / 1.5
        for i in range(-(-totals[s] // page)):
            table[s, i] = perm.pop()
            lo, hi = i * page, min((i + 1) * page, totals[s])
            kc[table[s, i], :hi - lo] = k[lo:hi]
            vc[table[s, i], :hi - lo] = v[lo:hi]
        qs.append(q)
        refs.append(plain_causal_attention(q.float(), k.float(), v.float(), D ** -0.5, window=window or None))
    q_all = torch.cat(qs)
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    tile_seq, tile_row0 = tiles_for(np.array(q_lens, dtype=np.int32), G)
    seq_of = torch.repeat_interleave(torch.arange(S, dtype=torch.int32), torch.tensor(q_lens))
    dev = lambda t: t.to(DEV)
    return dict(q=dev(q_all), kc=dev(kc), vc=dev(vc), table=dev(table), cu=dev(cu),
                before=dev(torch.tensor(befores, dtype=torch.int32)), tile_seq=dev(torch.from_numpy(tile_seq)),
                tile_row0=dev(torch.from_numpy(tile_row0)), n_tiles=len(tile_seq), seq_of=dev(seq_of),
                ref=torch.cat(refs))
