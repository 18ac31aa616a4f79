"""The step function's packing (csrc/host/step_pack.hpp), on the CPU: the packed arrays against a restatement in
numpy, for random mixtures of prompt portions and lone tokens; the attention work lists; what it refuses."""
import numpy as np
import pytest

from ai_engine_b200.cache import host


def manager(groups, max_seqs=8, max_pages=64):
    h = host()
    return h.CacheManager([h.GroupSpec(p, n, w) for p, n, w in groups], max_seqs, max_pages)


def segments(packed, lengths):
    out, o = [], 0
    for n in lengths:
        out.append(np.asarray(packed[o:o + n]))
        assert o % 4 == 0
        o += (n + 3) // 4 * 4
    assert o == len(packed) or len(packed) == 4
    return out


@pytest.mark.parametrize("seed", range(6))
def test_packed_arrays_against_numpy(seed):
    r = np.random.RandomState(seed)
    page = int(r.choice([8, 16]))
    c = manager([(page, 400, 0), (page, 400, 0)], max_seqs=8, max_pages=40)
    R = int(r.randint(1, 8))
    slots, starts, tokens, wants, srcs = [], [], [], [], []
    for _ in range(R):
        s = c.admit()
        start = int(r.randint(0, 200))
        n = 1 if r.rand() < 0.4 else int(r.randint(2, 70))
        assert c.ensure(s, start + n)
        slots.append(s)
        starts.append(start)
        tokens.append([int(x) for x in r.randint(0, 50000, size=n)])
        wants.append(sorted(set(int(x) for x in r.randint(0, n, size=r.randint(0, 4)))))
        srcs.append(int(r.randint(0, 8)) if n == 1 and r.rand() < 0.5 else -1)
    n_live = -1 if seed % 2 else max(1, R - 1)
    packed, lengths, T, Rr, N, max_q, max_total, width, has_src = host().pack_step(
        c, slots, starts, tokens, wants, srcs, n_live, page, bool(seed % 3 == 0))
    q_len = np.array([len(t) for t in tokens])
    assert (T, Rr, N) == (int(q_len.sum()), R, sum(len(w) for w in wants))
    assert max_q == q_len.max() and max_total == int((np.array(starts) + q_len).max())
    need = max(1, -(-max_total // page))
    assert width == (max(64, 1 << (need - 1).bit_length()) if seed % 3 == 0 else need)
    assert has_src == any(s >= 0 for s in srcs)
    (token_ids, positions, token_req, q_start, ql, ctx_len, sl, live, logit_rows, token_src, bt0, bt1) = segments(packed, lengths)
    want_start = np.concatenate([[0], np.cumsum(q_len)[:-1]])
    assert np.array_equal(q_start, want_start) and np.array_equal(ql, q_len)
    assert np.array_equal(ctx_len, starts) and np.array_equal(sl, slots)
    assert np.array_equal(live, [1 if (n_live < 0 or i < n_live) else 0 for i in range(R)])
    assert np.array_equal(token_ids, np.concatenate(tokens))
    assert np.array_equal(token_req, np.repeat(np.arange(R), q_len))
    assert np.array_equal(positions, np.concatenate([np.arange(s, s + n) for s, n in zip(starts, q_len)]))
    assert np.array_equal(logit_rows, [int(want_start[i]) + w for i in range(R) for w in wants[i]])
    src_want = np.full(T, -1)
    for i in range(R):
        if srcs[i] >= 0:
            src_want[want_start[i]] = srcs[i]
    assert np.array_equal(token_src, src_want)
    for g, bt in enumerate((bt0, bt1)):
        bt = bt.reshape(R, width)
        for i, s in enumerate(slots):
            pages = c.pages(g, s)
            assert list(bt[i, :len(pages)]) == pages and (bt[i, len(pages):] == -1).all()


def test_entries_that_are_refused():
    c = manager([(16, 8, 0)])
    s = c.admit()
    pack = lambda **kw: host().pack_step(c, kw.get("slots", [s]), kw.get("starts", [0]), kw.get("tokens", [[1, 2]]),
                                         kw.get("wants", [[]]), kw.get("srcs", [-1]), -1, 16, False)
    with pytest.raises(ValueError, match="at least one entry"):
        host().pack_step(c, [], [], [], [], [], -1, 16, False)
    with pytest.raises(ValueError, match="at least one token"):
        pack(tokens=[[]])
    with pytest.raises(ValueError, match="wanted place 2 is outside the entry's 2 tokens"):
        pack(wants=[[2]])
    with pytest.raises(ValueError, match="only an entry of one token"):
        pack(srcs=[0])
    with pytest.raises(ValueError, match="non-negative 32-bit"):
        pack(tokens=[[1, -5]])
    with pytest.raises(ValueError, match="non-negative 32-bit"):
        pack(tokens=[[1, 2 ** 31]])
    assert pack()[2:5] == (2, 1, 0)


def test_attention_work_lists():
    i32 = lambda a: np.asarray(a, dtype=np.int32)
    # requests: a lone token after 50, a portion of 300 after 10, a lone token after 900, a portion of 130 after 0
    q_len, ctx_len = i32([1, 300, 1, 130]), i32([50, 10, 900, 0])
    q_start = i32([0, 1, 301, 302])
    dec, other, tiles, pairs, n_decode, max_decode_len = host().attention_lists(q_start, q_len, ctx_len, 128)
    assert list(dec) == [301, 0] and n_decode == 2 and max_decode_len == 901      # the longest context first
    assert list(other) == list(range(1, 301)) + list(range(302, 432))
    # tiles by the keys before them, fewest first; units of two tiles are the tiles at even places of their request
    assert tiles.tolist() == [[3, 0], [1, 0], [3, 128], [1, 128], [1, 256]]
    assert pairs.tolist() == [[3, 0], [1, 0], [1, 256]]
    dec, other, tiles, pairs, n_decode, max_decode_len = host().attention_lists(i32([0, 1]), i32([1, 1]), i32([7, 7]), 128)
    assert list(dec) == [0, 1] and len(other) == 0 and tiles.shape == (0, 2) and pairs.shape == (0, 2)
    assert (n_decode, max_decode_len) == (2, 8)
