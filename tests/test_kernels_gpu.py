"""Each kernel alone against a plain PyTorch float32/float64 restatement of the same
op, at sizes other than the engine's tiny configurations."""
import math

import numpy as np
import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = "cuda"


def ops():
    from ai_engine_b200.kernels import ops as o
    return o


def err_word():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("D", [512, 2048, 3072, 4096])
@pytest.mark.parametrize("delta_kind", ["none", "bf16", "f32"])
def test_add_rmsnorm_many_rows(D, delta_kind):
    """Portions of prompts: hundreds of rows take a kernel of their own (four float4 per thread)."""
    torch.manual_seed(D)
    n = 300
    x = torch.randn(n, D, device=DEV) * 3
    delta = None if delta_kind == "none" else torch.randn(n, D, device=DEV).to(torch.bfloat16 if delta_kind == "bf16" else torch.float32)
    w = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16()
    s = x.double() + (delta.double() if delta is not None else 0)
    want = pl.rms_norm(s, w.double(), 1e-5)
    x_in = x.clone()
    out = ops().add_rmsnorm(x_in, delta, w, 1e-5, torch.bfloat16)
    assert torch.allclose(x_in.double(), s, atol=1e-6)
    assert (out.double() - want).abs().max() <= 2e-2 * max(1.0, float(want.abs().max()))
    rows = torch.arange(n - 1, -1, -1, device=DEV, dtype=torch.int32)
    out2 = ops().add_rmsnorm(x.clone(), None, w, 1e-5, torch.bfloat16, rows=rows, write_back=False)
    want2 = pl.rms_norm(x.double().flip(0), w.double(), 1e-5)
    assert (out2.double() - want2).abs().max() <= 2e-2 * max(1.0, float(want2.abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V,D", [(77, 24), (1000, 4096), (130, 200)])
def test_embed_gather(dtype, V, D):
    torch.manual_seed(0)
    table = torch.randn(V, D, device=DEV).to(dtype)
    ids = torch.randint(0, V, (19,), device=DEV, dtype=torch.int32)
    e = err_word()
    x = ops().embed_gather(ids, table, e)
    assert x.dtype == torch.float32 and torch.equal(x, table[ids.long()].float())
    assert int(e.item()) == 0
    bad = ids.clone()
    bad[3] = V
    x = ops().embed_gather(bad, table, e)
    assert int(e.item()) & 1 and torch.all(x[3] == 0)       # flagged, not trapped


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D,eps", [(48, 1e-5), (4096, 1e-6), (1000, 1e-3), (8200, 1e-5)])
def test_add_rmsnorm(dtype, D, eps):
    torch.manual_seed(1)
    n = 13
    x = torch.randn(n, D, device=DEV) * 3
    delta = torch.randn(n, D, device=DEV).to(dtype)
    w = (1 + 0.1 * torch.randn(D, device=DEV)).to(dtype)
    s = x.double() + delta.double()
    want = pl.rms_norm(s, w.double(), eps)
    x_in = x.clone()
    out = ops().add_rmsnorm(x_in, delta, w, eps, dtype)
    assert torch.allclose(x_in.double(), s, atol=1e-6)      # the sum was stored back in float32
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (out.double() - want).abs().max() <= tol * max(1.0, float(want.abs().max()))
    # without a pending branch, at chosen rows, not stored back
    rows = torch.tensor([5, 0, 12], device=DEV, dtype=torch.int32)
    x2 = x.clone()
    out2 = ops().add_rmsnorm(x2, None, w, eps, dtype, rows=rows, write_back=False)
    want2 = pl.rms_norm(x.double()[rows.long()], w.double(), eps)
    assert torch.equal(x2, x) and (out2.double() - want2).abs().max() <= tol * max(1.0, float(want2.abs().max()))
    # a 32-bit weight under bfloat16 activations stays 32-bit
    out3 = ops().add_rmsnorm(x.clone(), delta, w.float(), eps, dtype)
    assert (out3.double() - want).abs().max() <= tol * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,F", [(1, 24), (7, 1000), (33, 14336)])
def test_silu_mul(dtype, T, F):
    torch.manual_seed(2)
    gu = (torch.randn(T, 2 * F, device=DEV) * 2).to(dtype)
    g, u = gu[:, :F].double(), gu[:, F:].double()
    want = g * torch.sigmoid(g) * u
    out = ops().silu_mul(gu)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (out.double() - want).abs().max() <= tol * max(1.0, float(want.abs().max()))
    if F % 8 == 0:      # groups of 8 gate columns followed by their 8 up columns
        inter = torch.stack([gu[:, :F].reshape(T, -1, 8), gu[:, F:].reshape(T, -1, 8)], dim=2).reshape(T, 2 * F)
        out2 = ops().silu_mul(inter.contiguous(), block=8)
        assert torch.equal(out2, out)


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (5, 70, 33), (64, 64, 16), (130, 257, 1000), (3, 128256, 64)])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_gemm_f32_is_true_float32(M, N, K, wdtype):
    torch.manual_seed(3)
    a = torch.randn(M, K, device=DEV)
    w = torch.randn(N, K, device=DEV).to(wdtype)
    want = a.double() @ w.double().T
    out = ops().gemm_f32(a, w)
    assert (out.double() - want).abs().max() <= 2e-6 * K ** 0.5 * max(1.0, float(want.abs().max()))
    # a row's result does not depend on the other rows of the batch
    one = ops().gemm_f32(a[M // 2: M // 2 + 1].contiguous(), w)
    assert torch.equal(one[0], out[M // 2])
    # chosen rows
    rows = torch.tensor([M - 1, 0], device=DEV, dtype=torch.int32)
    sel = ops().gemm_f32(a, w, rows=rows)
    assert torch.equal(sel, out[rows.long()])


def paged_setup(dtype, H, K, d, P, lens, q_lens, seed, num_pages=None, shuffle=True):
    """Random q/k/v for requests with `lens` tokens in total, of which the last
    q_lens are this step's queries; pages scattered through the pool."""
    rng = np.random.RandomState(seed)
    torch.manual_seed(seed)
    R = len(lens)
    pages_per = [(n + P - 1) // P for n in lens]
    num_pages = num_pages or sum(pages_per) + 3
    perm = rng.permutation(num_pages) if shuffle else np.arange(num_pages)
    W = max(pages_per)
    bt = -np.ones((R, W), dtype=np.int32)
    at = 0
    for r, n in enumerate(pages_per):
        bt[r, :n] = perm[at:at + n]
        at += n
    k_pages = torch.full((num_pages, K, P, d), float("nan"), device=DEV, dtype=dtype)
    v_pages = torch.full((num_pages, K, P, d), float("nan"), device=DEV, dtype=dtype)
    ks = [(torch.randn(n, K, d, device=DEV) * 1.5).to(dtype) for n in lens]
    vs = [torch.randn(n, K, d, device=DEV).to(dtype) for n in lens]
    for r, n in enumerate(lens):
        for pos in range(n):
            pg, sl = bt[r, pos // P], pos % P
            k_pages[pg, :, sl] = ks[r][pos]
            v_pages[pg, :, sl] = vs[r][pos]
    T = sum(q_lens)
    q = torch.randn(T, H, d, device=DEV).to(dtype)
    positions, token_req = [], []
    for r, (n, ql) in enumerate(zip(lens, q_lens)):
        positions += list(range(n - ql, n))
        token_req += [r] * ql
    return dict(q=q, k_pages=k_pages, v_pages=v_pages, ks=ks, vs=vs,
                positions=torch.tensor(positions, device=DEV, dtype=torch.int32),
                token_req=torch.tensor(token_req, device=DEV, dtype=torch.int32),
                bt=torch.tensor(bt, device=DEV), lens=lens, q_lens=q_lens)


def paged_setup_fast(dtype, H, K, d, P, lens, q_lens, seed):
    """paged_setup without its loop over positions (for many or long requests)."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    R = len(lens)
    pages_per = [(n + P - 1) // P for n in lens]
    num_pages = sum(pages_per) + 3
    perm = torch.randperm(num_pages, generator=g, device=DEV)
    bt = -torch.ones((R, max(pages_per)), dtype=torch.int32, device=DEV)
    k_pages = torch.full((num_pages, K, P, d), float("nan"), device=DEV, dtype=dtype)
    v_pages = torch.full_like(k_pages, float("nan"))
    ks, vs, at = [], [], 0
    for r, n in enumerate(lens):
        bt[r, :pages_per[r]] = perm[at:at + pages_per[r]].int()
        at += pages_per[r]
        ks.append((torch.randn(n, K, d, generator=g, device=DEV) * 1.5).to(dtype))
        vs.append(torch.randn(n, K, d, generator=g, device=DEV).to(dtype))
        pos = torch.arange(n, device=DEV)
        k_pages[bt[r, pos // P].long(), :, pos % P] = ks[r]
        v_pages[bt[r, pos // P].long(), :, pos % P] = vs[r]
    q = torch.randn(sum(q_lens), H, d, generator=g, device=DEV).to(dtype)
    positions, token_req = [], []
    for r, (n, ql) in enumerate(zip(lens, q_lens)):
        positions += list(range(n - ql, n))
        token_req += [r] * ql
    return dict(q=q, k_pages=k_pages, v_pages=v_pages, ks=ks, vs=vs,
                positions=torch.tensor(positions, device=DEV, dtype=torch.int32),
                token_req=torch.tensor(token_req, device=DEV, dtype=torch.int32), bt=bt, lens=lens, q_lens=q_lens)


def attention_reference(s, H, K, d, scale, window):
    """[T, H, d] in float64 from the unpaged keys and values."""
    out = []
    t = 0
    for r, (n, ql) in enumerate(zip(s["lens"], s["q_lens"])):
        k = s["ks"][r].double().repeat_interleave(H // K, dim=1)       # [n, H, d]
        v = s["vs"][r].double().repeat_interleave(H // K, dim=1)
        for i in range(ql):
            pos = n - ql + i
            q = s["q"][t].double()                                      # [H, d]
            sc = torch.einsum("hd,nhd->hn", q, k) * scale
            j = torch.arange(n, device=DEV)
            ok = j <= pos
            if window:
                ok &= j > pos - window
            sc = sc.masked_fill(~ok[None], float("-inf"))
            out.append(torch.einsum("hn,nhd->hd", torch.softmax(sc, -1), v))
            t += 1
    return torch.stack(out)


ATTN_SHAPES = [  # H, K, d, P, lens, q_lens, window
    (4, 2, 16, 16, [5, 40], [5, 1], 0),
    (5, 1, 32, 8, [1, 9, 120], [1, 2, 120], 0),
    (6, 3, 48, 16, [300, 17], [1, 17], 0),
    (8, 8, 64, 4, [33, 64, 2], [3, 64, 1], 0),
    (32, 8, 128, 16, [700, 130], [1, 2], 0),
    (2, 1, 256, 32, [45], [45], 0),
    (4, 2, 80, 16, [150, 60], [150, 1], 37),
    (3, 1, 16, 8, [260], [1], 100),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", ATTN_SHAPES)
def test_paged_attention_plain(dtype, shape):
    H, K, d, P, lens, q_lens, window = shape
    s = paged_setup(dtype, H, K, d, P, lens, q_lens, seed=H * 100 + d)
    scale = 1.0 / math.sqrt(d)
    e = err_word()
    out = ops().paged_attention_plain(s["q"], s["k_pages"], s["v_pages"], s["positions"], s["token_req"],
                                      s["bt"], scale, window, e)
    want = attention_reference(s, H, K, d, scale, window)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert int(e.item()) == 0
    assert not torch.isnan(out).any()
    assert (out.double() - want).abs().max() <= tol


DECODE_SHAPES = [  # H, K, d, P, lens (one query each, the last token), window, splits
    (4, 1, 64, 16, [1, 40, 700], 0, 1),
    (32, 8, 128, 16, [1024, 3, 517, 90], 0, 4),
    (6, 2, 64, 8, [33, 257], 0, 3),
    (5, 1, 128, 16, [300, 31], 0, 2),          # a group of 5
    (8, 1, 64, 32, [129], 0, 7),               # more splits than 32-key tiles in places
    (2, 2, 128, 4, [64, 65, 1], 0, 1),
    (8, 2, 128, 16, [900, 40], 100, 3),        # window
    (24, 8, 128, 16, [2100], 0, 16),
    (16, 1, 64, 16, [77, 400], 0, 2),          # a group of 16: two CTAs of 8 heads per kv head
    (10, 1, 128, 8, [530], 0, 5),              # a group of 10: 8 + 2
]


@pytest.mark.parametrize("shape", DECODE_SHAPES)
def test_paged_attention_decode_split_kv(shape):
    H, K, d, P, lens, window, splits = shape
    s = paged_setup(torch.bfloat16, H, K, d, P, lens, [1] * len(lens), seed=H + d + splits)
    scale = 1.0 / math.sqrt(d)
    e = err_word()
    out = torch.full_like(s["q"], float("nan"))
    dec = torch.arange(len(lens), device=DEV, dtype=torch.int32)
    ops().paged_attention_decode(s["q"], s["k_pages"], s["v_pages"], dec, s["positions"], s["token_req"],
                                 s["bt"], scale, window, splits, e, out)
    want = attention_reference(s, H, K, d, scale, window)
    assert int(e.item()) == 0 and not torch.isnan(out).any()
    assert (out.double() - want).abs().max() <= 2e-2
    # the parts joined by the CTA that finishes last instead of by a second kernel: the same sums
    out2 = torch.full_like(s["q"], float("nan"))
    ops().paged_attention_decode(s["q"], s["k_pages"], s["v_pages"], dec, s["positions"], s["token_req"],
                                 s["bt"], scale, window, splits, e, out2, join_in_kernel=True)
    assert torch.equal(out2, out)
    # and again: the tickets of the first call are back at zero
    out3 = torch.full_like(s["q"], float("nan"))
    ops().paged_attention_decode(s["q"], s["k_pages"], s["v_pages"], dec, s["positions"], s["token_req"],
                                 s["bt"], scale, window, splits, e, out3, join_in_kernel=True)
    assert torch.equal(out3, out)


MANY_SHAPES = [  # H, K, d, P, lens, window, splits
    (32, 8, 64, 16, [2600, 130, 4095, 17, 900, 1, 16, 15, 33, 2048] * 6, 0, 1),      # 60 requests of mixed lengths
    (32, 8, 64, 16, [2600, 130, 4095, 17, 900, 1, 16, 15, 33, 2048] * 2, 0, 37),     # more parts than some requests have tiles
    (8, 2, 128, 64, [700, 64, 65, 1000], 0, 3),                                      # pages of 64
    (8, 2, 64, 8, [500, 90, 31], 60, 2),                                             # a window that starts mid-tile
    (20, 2, 128, 16, [333, 20], 0, 64),                                              # a group of 10; the most parts
]


@pytest.mark.parametrize("shape", MANY_SHAPES)
def test_paged_attention_decode_many_requests_and_parts(shape):
    H, K, d, P, lens, window, splits = shape
    s = paged_setup_fast(torch.bfloat16, H, K, d, P, lens, [1] * len(lens), seed=H + d + len(lens))
    scale = 1.0 / math.sqrt(d)
    e = err_word()
    want = attention_reference(s, H, K, d, scale, window)
    # a subset of the step's tokens, in another order; rows that are not asked for are not written
    pick = torch.tensor(list(range(len(lens)))[::-2], device=DEV, dtype=torch.int32)
    out = torch.full_like(s["q"], float("nan"))
    ops().paged_attention_decode(s["q"], s["k_pages"], s["v_pages"], pick, s["positions"], s["token_req"], s["bt"],
                                 scale, window, splits, e, out)
    torch.cuda.synchronize()
    assert int(e.item()) == 0
    err = (out[pick.long()].double() - want[pick.long()]).abs().amax(dim=(1, 2))
    assert err.max() <= 2e-2, f"first wrong request {int(pick[int((err > 2e-2).nonzero()[0])])}: {float(err.max())}"
    rest = torch.ones(len(lens), dtype=torch.bool, device=DEV)
    rest[pick.long()] = False
    assert torch.isnan(out[rest]).all()


PREFILL_SHAPES = [  # H, K, d, P, lens, q_lens, window
    (4, 2, 64, 16, [5, 40], [5, 7], 0),
    (32, 8, 128, 16, [300, 130, 64], [300, 2, 64], 0),
    (6, 2, 64, 8, [257, 65], [129, 65], 0),           # a portion that starts mid-page and mid-tile
    (5, 1, 128, 4, [700], [63], 0),
    (2, 2, 128, 32, [1100], [1100], 0),
    (8, 2, 64, 16, [400, 90], [400, 30], 70),         # window
    (3, 3, 128, 16, [200], [2], 0),
    (4, 1, 64, 64, [191, 192, 193], [191, 128, 2], 0),
]


@pytest.mark.parametrize("shape", PREFILL_SHAPES)
def test_paged_attention_prefill_tensor_cores(shape):
    H, K, d, P, lens, q_lens, window = shape
    s = paged_setup(torch.bfloat16, H, K, d, P, lens, q_lens, seed=H + d + len(lens))
    scale = 1.0 / math.sqrt(d)
    e = err_word()
    out = torch.full_like(s["q"], float("nan"))
    i32 = lambda a: torch.tensor(a, device=DEV, dtype=torch.int32)
    q_start = np.concatenate([[0], np.cumsum(q_lens)[:-1]])
    tiles = [(r, o) for r, n in enumerate(q_lens) for o in range(0, n, ops().PREFILL_TILE)]
    ops().paged_attention_prefill(s["q"], s["k_pages"], s["v_pages"], i32(tiles), i32(q_start), i32(q_lens),
                                  i32([n - ql for n, ql in zip(lens, q_lens)]), s["bt"], scale, window, e, out)
    want = attention_reference(s, H, K, d, scale, window)
    assert int(e.item()) == 0 and not torch.isnan(out).any()
    err = (out.double() - want).abs().amax(dim=(1, 2))
    assert err.max() <= 2e-2, f"first wrong token {int((err > 2e-2).nonzero()[0])} of {sum(q_lens)}: {float(err.max())}"


PREFILL_TC_SHAPES = [  # H, K, P, lens, q_lens  (head sizes 64 and 128, no window)
    (4, 2, 16, [5, 40], [5, 7]),
    (32, 8, 16, [300, 130, 64], [300, 2, 64]),
    (6, 2, 8, [257, 65], [129, 65]),           # a portion that starts mid-page and mid-tile
    (5, 1, 8, [700], [63]),
    (2, 2, 32, [1100], [1100]),
    (3, 3, 16, [200], [2]),
    (4, 1, 64, [191, 192, 193], [191, 128, 2]),
    (8, 2, 128, [128, 129, 384], [128, 129, 128]),
    (3, 1, 16, [256, 257, 255, 640], [256, 257, 255, 513]),      # units of two tiles: whole, one row over, one short
    (2, 1, 16, [1000, 1500], [300, 900]),                        # portions that start off a tile's edge, many key tiles
    (4, 4, 8, [77 + 384, 128 + 130], [384, 130]),
]


def prefill_work(q_lens, pair):
    """(request row, offset) of every tile of 128 tokens, or of every unit of two tiles."""
    step = 256 if pair else 128
    return [(r, o) for r, n in enumerate(q_lens) for o in range(0, n, step)]


@pytest.mark.parametrize("pair", [False, True], ids=["one_tile", "two_tiles"])
@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("shape", PREFILL_TC_SHAPES)
def test_paged_attention_prefill_tcgen05(shape, d, pair):
    H, K, P, lens, q_lens = shape
    s = paged_setup(torch.bfloat16, H, K, d, P, lens, q_lens, seed=H + P + len(lens))
    scale = 1.0 / math.sqrt(d)
    e = err_word()
    out = torch.full_like(s["q"], float("nan"))
    i32 = lambda a: torch.tensor(a, device=DEV, dtype=torch.int32)
    q_start = np.concatenate([[0], np.cumsum(q_lens)[:-1]])
    took = ops().paged_attention_prefill_tc(s["q"], s["k_pages"], s["v_pages"], i32(prefill_work(q_lens, pair)),
                                            i32(q_start), i32(q_lens), i32([n - ql for n, ql in zip(lens, q_lens)]),
                                            s["bt"], scale, 0, e, out, pair=pair)
    assert took
    torch.cuda.synchronize()
    assert int(e.item()) == 0, "a bounded wait ran out or a page was missing"
    want = attention_reference(s, H, K, d, scale, 0)
    assert not torch.isnan(out).any()
    err = (out.double() - want).abs().amax(dim=(1, 2))
    assert err.max() <= 2e-2, f"first wrong token {int((err > 2e-2).nonzero()[0])} of {sum(q_lens)}: {float(err.max())}"


@pytest.mark.parametrize("pair", [False, True], ids=["one_tile", "two_tiles"])
def test_prefill_tcgen05_scores_that_grow_along_the_sequence(pair):
    """Keys whose size grows from tile to tile (scores up to tens of units above everything before) and
    then falls again: rows whose reference maximum has to move, and rows where it may stay."""
    H, K, d, P = 6, 2, 128, 16
    n = 900
    s = paged_setup(torch.bfloat16, H, K, d, P, [n], [n], seed=21)
    gain = torch.ones(n, device=DEV)
    gain[130:260], gain[260:520], gain[520:700] = 2.0, 6.0, 0.3
    for pos in range(n):
        s["ks"][0][pos] = (s["ks"][0][pos].float() * gain[pos]).bfloat16()
        pg, sl = int(s["bt"][0, pos // P]), pos % P
        s["k_pages"][pg, :, sl] = s["ks"][0][pos]
    scale = 1.0 / math.sqrt(d)
    e = err_word()
    out = torch.full_like(s["q"], float("nan"))
    i32 = lambda a: torch.tensor(a, device=DEV, dtype=torch.int32)
    assert ops().paged_attention_prefill_tc(s["q"], s["k_pages"], s["v_pages"], i32(prefill_work([n], pair)), i32([0]),
                                            i32([n]), i32([0]), s["bt"], scale, 0, e, out, pair=pair)
    torch.cuda.synchronize()
    assert int(e.item()) == 0
    want = attention_reference(s, H, K, d, scale, 0)
    err = (out.double() - want).abs().amax(dim=(1, 2))
    assert err.max() <= 2e-2, f"first wrong token {int((err > 2e-2).nonzero()[0])} of {n}: {float(err.max())}"


def test_prefill_tcgen05_refuses_what_it_does_not_take():
    s = paged_setup(torch.bfloat16, 4, 2, 32, 16, [40], [40], seed=1)
    i32 = lambda a: torch.tensor(a, device=DEV, dtype=torch.int32)
    out = torch.zeros_like(s["q"])
    args = (s["q"], s["k_pages"], s["v_pages"], i32([[0, 0]]), i32([0]), i32([40]), i32([0]), s["bt"], 0.125)
    assert not ops().paged_attention_prefill_tc(*args, 0, err_word(), out)          # head size 32
    s = paged_setup(torch.bfloat16, 4, 2, 128, 16, [40], [40], seed=1)
    args = (s["q"], s["k_pages"], s["v_pages"], i32([[0, 0]]), i32([0]), i32([40]), i32([0]), s["bt"], 0.09)
    assert not ops().paged_attention_prefill_tc(*args, 7, err_word(), torch.zeros_like(s["q"]))   # a window
    s = paged_setup(torch.bfloat16, 4, 2, 128, 4, [40], [40], seed=1)
    args = (s["q"], s["k_pages"], s["v_pages"], i32([[0, 0]]), i32([0]), i32([40]), i32([0]), s["bt"], 0.09)
    assert not ops().paged_attention_prefill_tc(*args, 0, err_word(), torch.zeros_like(s["q"]))   # pages of 4 keys


def test_mixed_step_decode_and_prefill_kernels_side_by_side():
    """A mixed step: requests 0 and 2 bring one token, request 1 brings five."""
    H, K, d, P = 8, 2, 64, 16
    s = paged_setup(torch.bfloat16, H, K, d, P, [70, 30, 200], [1, 5, 1], seed=3)
    scale = 1.0 / math.sqrt(d)

    class Ctx:
        pass

    ctx = Ctx()
    ctx.positions, ctx.token_req, ctx.err = s["positions"], s["token_req"], err_word()
    ctx.n_decode, ctx.max_decode_len = 2, 200
    ctx.decode_tokens = torch.tensor([0, 6], device=DEV, dtype=torch.int32)
    ctx.other_tokens = torch.tensor([1, 2, 3, 4, 5], device=DEV, dtype=torch.int32)
    i32 = lambda a: torch.tensor(a, device=DEV, dtype=torch.int32)
    ctx.R, ctx.prefill_tiles = 3, i32([[1, 0]])
    ctx.q_start, ctx.q_len, ctx.ctx_len = i32([0, 1, 6]), i32([1, 5, 1]), i32([69, 25, 199])
    out = ops().paged_attention(s["q"], s["k_pages"], s["v_pages"], ctx, ctx, s["bt"], scale, 0)
    want = attention_reference(s, H, K, d, scale, 0)
    assert (out.double() - want).abs().max() <= 2e-2


def test_step_attention_with_the_two_tile_kernel(monkeypatch):
    """`paged_attention` with the rule that picks the prompt kernel turned to "two tiles": portions of three requests
    (one of them with a lone last tile, one shorter than a tile) beside a lone decoded token, work lists as the
    planner makes them."""
    H, K, d, P = 8, 2, 128, 16
    lens, q_lens = [700, 90, 300, 411], [520, 40, 1, 256]
    s = paged_setup(torch.bfloat16, H, K, d, P, lens, q_lens, seed=5)
    scale = 1.0 / math.sqrt(d)
    i32 = lambda a: torch.tensor(a, device=DEV, dtype=torch.int32)
    q_start = np.concatenate([[0], np.cumsum(q_lens)[:-1]])

    class Ctx:
        pass

    ctx = Ctx()
    ctx.positions, ctx.token_req, ctx.err = s["positions"], s["token_req"], err_word()
    ctx.R, ctx.n_decode, ctx.max_decode_len = 4, 1, 300
    ctx.decode_tokens = i32([int(q_start[2])])
    ctx.prefill_tiles = i32([(r, o) for r in (0, 1, 3) for o in range(0, q_lens[r], 128)])
    ctx.prefill_pairs = i32([(r, o) for r in (0, 1, 3) for o in range(0, q_lens[r], 256)])
    ctx.q_start, ctx.q_len, ctx.ctx_len = i32(q_start), i32(q_lens), i32([n - q for n, q in zip(lens, q_lens)])
    want = attention_reference(s, H, K, d, scale, 0)
    asked = []
    monkeypatch.setattr(ops(), "prefill_takes_pairs", lambda *a: asked.append(a) or True)
    out = ops().paged_attention(s["q"], s["k_pages"], s["v_pages"], ctx, ctx, s["bt"], scale, 0)
    torch.cuda.synchronize()
    assert asked == [(8, 5, H)] and int(ctx.err.item()) == 0
    err = (out.double() - want).abs().amax(dim=(1, 2))
    assert err.max() <= 2e-2, f"first wrong token {int((err > 2e-2).nonzero()[0])}: {float(err.max())}"


def test_the_rule_that_picks_the_prompt_kernel(monkeypatch):
    monkeypatch.setattr(ops(), "sm_count", lambda: 148)
    takes = ops().prefill_takes_pairs
    assert takes(16, 8, 32)            # 2,048 tokens of one request, 32 heads: 256 CTAs against 512
    assert takes(64, 32, 8)
    assert not takes(16, 8, 24)        # 192 CTAs would run in two uneven rounds
    assert not takes(8, 4, 32)         # fewer CTAs than SMs: the longest decides
    assert not takes(16, 16, 32)       # every unit holds one tile only
    assert not takes(0, 0, 32)


def test_far_key_among_hundreds_is_found():
    """One key far back is made to match the query; the output must be its value."""
    H, K, d, P = 4, 2, 32, 16
    s = paged_setup(torch.float32, H, K, d, P, [600], [1], seed=9)
    far = 37
    pg, sl = int(s["bt"][0, far // P]), far % P
    s["k_pages"][pg, :, sl] = 0
    for h in range(H):
        s["k_pages"][pg, h // (H // K), sl] += s["q"][0, h] * 10 / (H // K)
    out = ops().paged_attention_plain(s["q"], s["k_pages"], s["v_pages"], s["positions"], s["token_req"],
                                      s["bt"], 1.0, 0, err_word())
    s["ks"][0][far] = s["k_pages"][pg, :, sl]
    want = attention_reference(s, H, K, d, 1.0, 0)
    assert (out.double() - want).abs().max() <= 2e-5
    assert (out[0, 0] - s["v_pages"][pg, 0, sl]).abs().max() < 0.2     # dominated by the far key's value


def test_bad_page_is_flagged_not_followed():
    s = paged_setup(torch.float32, 2, 1, 16, 8, [20], [1], seed=4)
    s["bt"][0, 1] = 10_000
    e = err_word()
    out = ops().paged_attention_plain(s["q"], s["k_pages"], s["v_pages"], s["positions"], s["token_req"],
                                      s["bt"], 1.0, 0, e)
    torch.cuda.synchronize()
    assert int(e.item()) & 2 and not torch.isnan(out).any()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,K,d,P,rot", [(4, 2, 16, 16, 16), (5, 1, 32, 8, 32), (6, 3, 48, 4, 32),
                                         (32, 8, 128, 16, 128), (2, 2, 64, 16, 0)])
@pytest.mark.parametrize("many", [False, True])
def test_rope_kv_write(dtype, H, K, d, P, rot, many):
    """many: enough tokens for the block-per-token kernel that portions of prompts take in bfloat16."""
    torch.manual_seed(5)
    lens, q_lens = ([130, 100, 3], [90, 40, 1]) if many else ([9, 41, 3], [9, 2, 1])
    s = paged_setup(dtype, H, K, d, P, lens, q_lens, seed=6)
    T = sum(q_lens)
    qkv = torch.randn(T, (H + 2 * K) * d, device=DEV).to(dtype)
    inv_freq = torch.from_numpy(pl.inv_freq_default(rot, 500000.0)).to(DEV) if rot else torch.zeros(0, device=DEV)
    before_k = s["k_pages"].clone()
    e = err_word()
    q = ops().rope_kv_write(qkv, s["k_pages"], s["v_pages"], s["positions"], s["token_req"], s["bt"],
                            inv_freq, H, K, d, e)
    assert int(e.item()) == 0
    x = qkv.double().view(T, H + 2 * K, d)
    pos = s["positions"].cpu()

    def rot_ref(t):     # [T, heads, d]
        if not rot:
            return t
        r = pl.rope(t[..., :rot].transpose(0, 1), pos, pl.inv_freq_default(rot, 500000.0)).transpose(0, 1)
        return torch.cat([r, t[..., rot:]], dim=-1)

    xq, xk, xv = x[:, :H].cpu(), x[:, H:H + K].cpu(), x[:, H + K:].cpu()
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert (q.double().cpu() - rot_ref(xq)).abs().max() <= tol * 4
    kr = rot_ref(xk)
    touched = torch.zeros_like(before_k, dtype=torch.bool)
    for t in range(T):
        r, p = int(s["token_req"][t]), int(pos[t])
        pg, sl = int(s["bt"][r, p // P]), p % P
        assert (s["k_pages"][pg, :, sl].double().cpu() - kr[t]).abs().max() <= tol * 4
        assert (s["v_pages"][pg, :, sl].double().cpu() - xv[t]).abs().max() <= tol
        touched[pg, :, sl] = True
    same = (s["k_pages"] == before_k) | (torch.isnan(s["k_pages"]) & torch.isnan(before_k))
    assert bool(same[~touched].all())           # nothing else in the pool was written
    # write=False leaves the pool alone and still rotates q
    k2 = s["k_pages"].clone()
    q2 = ops().rope_kv_write(qkv, s["k_pages"], s["v_pages"], s["positions"], s["token_req"], s["bt"],
                             inv_freq, H, K, d, e, write=False)
    assert torch.equal(q2, q) and bool(((s["k_pages"] == k2) | torch.isnan(k2)).all())


def test_take_sampled_ids_hands_tokens_over_on_the_device():
    """ids[t] = last[src[t]] where src[t] >= 0; the others stay; a source row outside `last` is flagged."""
    last = torch.tensor([11, 22, 33, 44], device=DEV, dtype=torch.int32)
    ids = torch.tensor([5, 0, 7, 0, 9, 0], device=DEV, dtype=torch.int32)
    src = torch.tensor([-1, 2, -1, 0, -1, 3], device=DEV, dtype=torch.int32)
    e = err_word()
    ops().take_sampled_ids(ids, src, last, e)
    assert ids.tolist() == [5, 33, 7, 11, 9, 44] and int(e.item()) == 0
    ops().take_sampled_ids(ids, torch.tensor([4, -1, -1, -1, -1, -1], device=DEV, dtype=torch.int32), last, e)
    torch.cuda.synchronize()
    assert int(e.item()) & 1 and ids.tolist() == [5, 33, 7, 11, 9, 44]


@pytest.mark.parametrize("N,V", [(1, 7), (8, 128256), (64, 1000), (3, 8192 * 5 + 13)])
def test_greedy_over_several_blocks_takes_the_first_maximum(N, V):
    from ai_engine_b200.sampling.sampler import argmax_rows

    torch.manual_seed(N + V)
    base = torch.randn(N, V + 5, device=DEV)
    logits = base[:, :V]                                   # rows V + 5 apart
    for r in range(N):                                      # ties at the maximum: the first one wins
        top = float(logits[r].max()) + 1.0
        where = torch.randperm(V, device=DEV)[:min(3, V)]
        logits[r, where] = top
    if N > 2:
        logits[1, :] = float("-inf")                        # no finite value: index 0
        logits[2, 0] = float("nan")                         # a NaN is never chosen
    scratch = (torch.zeros(64, dtype=torch.int64, device=DEV), torch.zeros(64, dtype=torch.int32, device=DEV))
    for _ in range(2):                                      # the scratch comes back zeroed
        got = argmax_rows(logits, scratch).cpu()
        assert int(scratch[0].abs().sum()) == 0 and int(scratch[1].abs().sum()) == 0
    want = []
    for r in range(N):
        row = logits[r].clone()
        row[torch.isnan(row)] = float("-inf")
        want.append(int((row == row.max()).nonzero()[0]))
    assert got.tolist() == want


def test_sampling_kernel_against_the_plain_sampler():
    from ai_engine_b200.sampling.sampler import sample_rows

    rng = np.random.RandomState(0)
    V = 1000
    cases = []
    for i in range(120):
        T = [0.0, 0.8, 1.0, 2.5][i % 4]
        k = [0, 0, 5, 50][(i // 4) % 4]
        p = [1.0, 0.9, 0.3, 1.0][(i // 16) % 4]
        cases.append((T, k, p, float(np.float32(rng.rand()))))
    logits = torch.randn(len(cases), V) * 2
    logits[7, 100] = logits[7].max() + 1            # ties for the maximum: the first wins
    logits[7, 10] = logits[7, 100]
    logits[8] = torch.round(logits[8] * 2) / 2      # many ties under temperature
    logits[9] = torch.round(logits[9])
    dev = lambda a, dt: torch.tensor(a, dtype=dt, device=DEV)
    out = sample_rows(logits.to(DEV), dev([c[0] for c in cases], torch.float32),
                      dev([c[1] for c in cases], torch.int32), dev([c[2] for c in cases], torch.float32),
                      dev([c[3] for c in cases], torch.float32)).cpu().tolist()
    wrong = []
    for i, (T, k, p, r) in enumerate(cases):
        want = pl.sample(logits[i].tolist(), T, top_k=k or None, top_p=p if p < 1 else None, r=r)
        if out[i] != want:
            # a draw that falls within float rounding of a boundary of the cumulative sum may
            # land on either neighbour; anything else is a fault
            near = {pl.sample(logits[i].tolist(), T, top_k=k or None, top_p=p if p < 1 else None, r=r2)
                    for r2 in (max(r - 2e-6, 0.0), min(r + 2e-6, 1.0))}
            if out[i] not in near:
                wrong.append((i, T, k, p, r, out[i], want))
    assert not wrong, wrong[:5]
    assert out[7] == 10 or cases[7][0] != 0.0


def test_sampling_distribution_and_large_vocab():
    from ai_engine_b200.sampling.sampler import sample_rows

    V, N = 128256, 64
    torch.manual_seed(1)
    base = torch.randn(V) * 3
    logits = base[None].repeat(N, 1).to(DEV)
    greedy = sample_rows(logits, torch.zeros(N, device=DEV), torch.zeros(N, dtype=torch.int32, device=DEV),
                         torch.ones(N, device=DEV), torch.zeros(N, device=DEV))
    assert greedy.tolist() == [int(base.argmax())] * N
    r = torch.linspace(0, 0.999, N, device=DEV)
    out = sample_rows(logits, torch.ones(N, device=DEV), torch.full((N,), 20, dtype=torch.int32, device=DEV),
                      torch.ones(N, device=DEV), r).cpu().tolist()
    top20 = set(torch.topk(base, 20).indices.tolist())
    assert set(out) <= top20
    # the walk is monotone: a larger draw never lands on a more likely token
    vals = [float(base[t]) for t in out]
    assert all(vals[i] >= vals[i + 1] - 1e-6 for i in range(N - 1))


@pytest.mark.parametrize("kind", ["decode", "prefill"])
def test_fast_kernels_find_a_far_key_and_respect_a_window_edge(kind):
    """One key far back matches the query exactly (score far above the rest): the output must be its
    value; with a window that ends one key after it, it must not be seen at all."""
    H, K, d, P, n, far = 8, 2, 128, 16, 700, 37
    q_len = 1 if kind == "decode" else 5
    s = paged_setup(torch.bfloat16, H, K, d, P, [n], [q_len], seed=21)
    pg, sl = int(s["bt"][0, far // P]), far % P
    s["q"][:] = s["q"] * 0.05
    s["k_pages"][pg, :, sl] = 0
    for h in range(H):      # the far key of each kv head points along the sum of its heads' queries
        s["k_pages"][pg, h // (H // K), sl] += (s["q"][q_len - 1, h].float() * 400).bfloat16()
    s["ks"][0][far] = s["k_pages"][pg, :, sl]
    i32 = lambda a: torch.tensor(a, device=DEV, dtype=torch.int32)

    def run(window):
        out = torch.full_like(s["q"], float("nan"))
        e = err_word()
        if kind == "decode":
            ops().paged_attention_decode(s["q"], s["k_pages"], s["v_pages"], i32([0]), s["positions"], s["token_req"],
                                         s["bt"], 1.0, window, 3, e, out)
        else:
            ops().paged_attention_prefill(s["q"], s["k_pages"], s["v_pages"], i32([[0, 0]]), i32([0]), i32([q_len]),
                                          i32([n - q_len]), s["bt"], 1.0, window, e, out)
        assert int(e.item()) == 0
        return out

    out = run(0)
    want = attention_reference(s, H, K, d, 1.0, 0)
    assert (out.double() - want).abs().max() <= 2e-2
    assert (out[q_len - 1, 0].float() - s["v_pages"][pg, 0, sl].float()).abs().max() < 0.1
    # the last query sits at n - 1: a window of n - 1 - far keys ends just after the far key
    w = n - 1 - far
    out_w = run(w)
    want_w = attention_reference(s, H, K, d, 1.0, w)
    assert (out_w.double() - want_w).abs().max() <= 2e-2
    assert (out_w[q_len - 1, 0].float() - s["v_pages"][pg, 0, sl].float()).abs().max() > 0.3
    out_w1 = run(w + 1)             # one key wider: the far key is back
    assert (out_w1[q_len - 1, 0].float() - s["v_pages"][pg, 0, sl].float()).abs().max() < 0.1
