"""The work list of the persistent attention kernel (csrc/flash_prefill_sm100.cu, `fa_item`),
restated in Python: every CTA derives its items from (round, blockIdx, gridDim) alone, so the three
roles of a CTA walk identical lists with no communication.  These checks pin the properties the
kernel relies on: every 128-row query tile of every (batch, head) is produced exactly once, key-tile
counts follow the causal rule, a stream without rows gets no tiles, and the alternating deal keeps
the causal load of the CTAs within one round of each other."""
import itertools

import pytest

BM = BN = 128


def fa_item(r, c, G, S, kv_len, q_pos0, n_q, batch, causal):
    """Mirror of the device function: work item of CTA c in round r, or None."""
    n_mp = (S + 2 * BM - 1) // (2 * BM)
    n_bh = n_q * batch
    n_items = n_mp * n_bh
    w = r * G + ((G - 1 - c) if (causal and (r & 1)) else c)
    if w >= n_items:
        return None
    if causal:
        mp, bh = n_mp - 1 - w // n_bh, w % n_bh
    else:
        mp, bh = w % n_mp, w // n_mp
    head, b, m0 = bh % n_q, bh // n_q, mp * 2 * BM
    kv0 = kv1 = kv_len
    if causal:
        kv0 = min(kv0, q_pos0 + m0 + BM)
        kv1 = min(kv1, q_pos0 + m0 + 2 * BM)
    n0 = (kv0 + BN - 1) // BN
    n1 = (kv1 + BN - 1) // BN if m0 + BM < S else 0
    return b, head, m0, n0, n1


CASES = [  # S, kv_len, q_pos0, n_q, batch, causal
    (512, 512, 0, 16, 64, False), (8192, 8192, 0, 32, 1, True), (1500, 1500, 0, 20, 1, False),
    (1024, 1024, 0, 32, 1, True), (130, 130, 0, 6, 3, False), (700, 700, 0, 8, 5, True),
    (4, 1500, 0, 20, 1, False), (64, 64, 0, 4, 1, True), (300, 812, 512, 8, 2, True),
]


@pytest.mark.parametrize("S,kv_len,q_pos0,n_q,batch,causal", CASES)
@pytest.mark.parametrize("sms", [148, 1, 7])
def test_every_query_tile_once_and_tile_counts(S, kv_len, q_pos0, n_q, batch, causal, sms):
    n_mp = (S + 2 * BM - 1) // (2 * BM)
    n_items = n_mp * n_q * batch
    G = min(n_items, sms)
    rounds = (n_items + G - 1) // G
    seen = {}
    for c, r in itertools.product(range(G), range(rounds)):
        it = fa_item(r, c, G, S, kv_len, q_pos0, n_q, batch, causal)
        if it is None:
            continue
        b, head, m0, n0, n1 = it
        assert n0 >= 1                                   # stream A always has rows and keys
        for x, n in ((0, n0), (1, n1)):
            rows0 = m0 + x * BM
            if rows0 >= S:
                assert n == 0                            # no rows: the stream stays idle
                continue
            key = (b, head, rows0)
            assert key not in seen, f"tile {key} produced twice"
            seen[key] = n
            last_key = min(kv_len, q_pos0 + rows0 + BM) if causal else kv_len
            assert n == (last_key + BN - 1) // BN        # exactly the tiles that hold visible keys
        assert n1 == 0 or n0 <= n1 <= n0 + 1             # the streams share every tile but the diagonal one
    n_mt = (S + BM - 1) // BM
    assert len(seen) == n_mt * n_q * batch


@pytest.mark.parametrize("S,n_q", [(8192, 32), (4096, 32), (4096, 64), (2048, 32)])
def test_causal_deal_is_balanced(S, n_q):
    """Heaviest first, dealt forwards and backwards in alternate rounds: the key tiles a CTA
    gets differ from the mean by less than one round's heaviest item (problems of at least two
    rounds: with fewer items than CTAs the longest item is the critical path whatever the deal)."""
    G = 148
    n_items = ((S + 255) // 256) * n_q
    rounds = (n_items + G - 1) // G
    load = []
    for c in range(G):
        tot = 0
        for r in range(rounds):
            it = fa_item(r, c, G, S, S, 0, n_q, 1, True)
            if it is not None:
                tot += it[3] + it[4]
        load.append(tot)
    heaviest = 2 * ((S + BN - 1) // BN)
    mean = sum(load) / G
    assert max(load) - mean < heaviest
    assert max(load) <= 1.08 * mean
