"""Correctness at the context lengths that the benchmark reports: 8,192 tokens at the layer sizes of
Llama-3-8B and 32,768 at those of Llama-3.2-3B with llama3 scaling, through the engine (one layer of the
full width and a reduced vocabulary, so that the plain implementation stays affordable: it computes keys
and values for every position and queries, feed-forward and logits only for the rows compared), and the
attention kernels alone at 33,000 keys (block tables of more than 2,000 entries, so that the decode kernel
must cut a request into more parts than the machine's size asks for) and for a prompt portion that follows
30,720 cached tokens.  Single far keys are made to match single queries, so that a page lost or misplaced
anywhere along the sequence shows."""
import math
import os

import numpy as np
import pytest
import torch

from helpers import TOL_BF16, plain_logits, random_ids
from test_replay_gpu import F32_FULL_WIDTH_TOL, FULL_SIZE_LAYERS

pytestmark = pytest.mark.gpu
DEV = "cuda"


def ops():
    from ai_engine_b200.kernels import ops as o
    return o


def one_layer_dir(tmp_path, name, max_pos):
    import ai_engine_b200 as aie

    raw = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=1, vocab_size=2048, rope_theta=500000.0,
               rms_norm_eps=1e-5, max_position_embeddings=max_pos, **FULL_SIZE_LAYERS[name])
    d = os.path.join(str(tmp_path), name)
    # projections of standard deviation 0.025 instead of 0.02: scores spread by 2.5 units, so that tens of
    # keys among thousands carry a row's weight and a missing page moves its logits
    aie.write_random_model(aie.LlamaConfig.from_dict(raw), d, seed=8, dtype="bfloat16", std=0.025)
    return d


def feed_and_compare(rep, d, seqs, tail, tol_of, odt, portion=2048):
    """Each request's prompt (all but its last `tail` tokens) alone in portions of `portion` tokens, then the
    last `tail` tokens of all requests side by side, one step a token.  Compared: the last (up to) 64 prompt
    rows and every decoded row."""
    got, rows_of = {}, {}
    for rid, ids in seqs.items():
        n = len(ids) - tail
        first = max(0, n - 64)
        rows_of[rid] = list(range(first, len(ids)))
        got[rid] = []
        for a in range(0, n, portion):
            b = min(a + portion, n)
            want = [r - a for r in range(max(first, a), b)]
            out = rep.run_step([dict(id=rid, tokens=ids[a:b], want=want)])
            if want:
                got[rid].append(out.numpy())
    for k in range(tail):
        out = rep.run_step([dict(id=rid, tokens=[ids[len(ids) - tail + k]], want=[0]) for rid, ids in seqs.items()]).numpy()
        for j, rid in enumerate(seqs):
            got[rid].append(out[j:j + 1])
    rep.run_step([], end=list(seqs))
    worst = 0.0
    for rid, ids in seqs.items():
        ref = plain_logits(d, ids, odt, rows=rows_of[rid])
        tol = tol_of(ref)
        err = np.abs(np.concatenate(got[rid]) - ref).max(axis=1)
        assert err.max() <= tol, (f"request {rid} of {len(ids)} tokens: first wrong row {rows_of[rid][int(np.argmax(err > tol))]}: "
                                  f"{err.max()} (gate {tol})")
        worst = max(worst, float(err.max() / tol))
    return worst


def test_llama3_8b_layer_at_8192_tokens(tmp_path):
    """Eight requests of 40 to 8,192 tokens: prompts in portions of 2,048 tokens (the tcgen05 prompt kernel
    walks up to 48 key tiles of earlier portions), then 32 tokens one by one, all eight side by side (the
    decode kernel over block tables of 512 entries beside short ones)."""
    from ai_engine_b200.engine.replay import Replayer

    d = one_layer_dir(tmp_path, "llama3_8b", 8192)
    lens = [8192, 8192, 5000, 3000, 2081, 1000, 300, 40]
    seqs = {f"r{i}": random_ids(n, 2048, 500 + i) for i, n in enumerate(lens)}
    rep = Replayer(d, "bfloat16", max_tokens=sum((n + 63) // 64 * 64 for n in lens), block_size=16, max_num_seqs=8)
    worst = feed_and_compare(rep, d, seqs, 32, lambda ref: TOL_BF16 * max(1.0, float(np.abs(ref).max())), torch.float32)
    print(f"8,192-token context, bfloat16: worst difference {worst:.2f} of its gate")
    assert rep.cache.book.pages_in_use(0) == 0
    # the 32-bit path at the same length (one request: its kernels are slow)
    rep = Replayer(d, "float32", max_tokens=8192, block_size=16, max_num_seqs=2)
    worst = feed_and_compare(rep, d, {"r0": seqs["r0"]}, 8,
                             lambda ref: F32_FULL_WIDTH_TOL * max(1.0, float(np.abs(ref).max())), torch.float64)
    print(f"8,192-token context, float32: worst difference {worst:.2f} of its gate")


def test_llama32_3b_layer_at_32768_tokens_with_llama3_scaling(tmp_path):
    """One request: a 32,768-token prompt in sixteen portions of 2,048, then 16 tokens one by one; rotation
    angles at positions up to 32,783 under llama3 scaling (factor 32, original 8,192)."""
    from ai_engine_b200.engine.replay import Replayer

    d = one_layer_dir(tmp_path, "llama32_3b", 40960)
    ids = random_ids(32768 + 16, 2048, 77)
    rep = Replayer(d, "bfloat16", max_tokens=32768 + 64, block_size=16, max_num_seqs=2)
    worst = feed_and_compare(rep, d, {"long": ids}, 16, lambda ref: TOL_BF16 * max(1.0, float(np.abs(ref).max())),
                             torch.float32)
    print(f"32,768-token context, bfloat16: worst difference {worst:.2f} of its gate")


# ---------------------------------------------------------------------------------------------------------
def long_request(H, K, d, P, n, n_q, seed, planted):
    """One request of n keys in pages scattered through the pool, the last n_q of them this step's queries.
    planted: (query row, far position) pairs; the key at the far position is made to match the first query head
    of every group of that row, so that this head's output is, to a few percent, the far key's value."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    pages = (n + P - 1) // P
    perm = torch.randperm(pages + 7, generator=g, device=DEV)
    bt = perm[:pages].to(torch.int32).view(1, -1).contiguous()
    ks = (torch.randn(n, K, d, generator=g, device=DEV) * 1.2).bfloat16()
    vs = torch.randn(n, K, d, generator=g, device=DEV).bfloat16()
    q = torch.randn(n_q, H, d, generator=g, device=DEV).bfloat16()
    G = H // K
    for row, far in planted:
        ks[far] = (q[row, ::G].float() * (22.0 / (d ** 0.5))).bfloat16()        # score near 22 * |q|^2 / d
    k_pages = torch.full((pages + 7, K, P, d), float("nan"), device=DEV, dtype=torch.bfloat16)
    v_pages = torch.full_like(k_pages, float("nan"))
    pos = torch.arange(n, device=DEV)
    k_pages[bt[0, pos // P].long(), :, pos % P] = ks
    v_pages[bt[0, pos // P].long(), :, pos % P] = vs
    return dict(q=q, ks=ks, vs=vs, k_pages=k_pages, v_pages=v_pages, bt=bt, n=n, n_q=n_q,
                positions=torch.arange(n - n_q, n, device=DEV, dtype=torch.int32),
                token_req=torch.zeros(n_q, device=DEV, dtype=torch.int32))


def long_reference(s, H, K, scale, chunk=128):
    """[n_q, H, d] in float64, a chunk of query rows at a time."""
    G = H // K
    k = s["ks"].double().repeat_interleave(G, dim=1)
    v = s["vs"].double().repeat_interleave(G, dim=1)
    j = torch.arange(s["n"], device=DEV)
    out = []
    for a in range(0, s["n_q"], chunk):
        q = s["q"][a:a + chunk].double()
        sc = torch.einsum("thd,nhd->thn", q, k) * scale
        pos = s["positions"][a:a + chunk].long()
        sc = sc.masked_fill(~(j[None, :] <= pos[:, None])[:, None, :], float("-inf"))
        out.append(torch.einsum("thn,nhd->thd", torch.softmax(sc, -1), v))
    return torch.cat(out)


@pytest.mark.parametrize("P,H,K,d", [(16, 32, 8, 128), (8, 8, 2, 64), (16, 24, 8, 128)])
def test_decode_attention_at_33000_keys(P, H, K, d):
    """A lone token over 33,000 cached keys: the block table has 2,063 (page 16) or 4,125 (page 8) entries, more
    than one CTA keeps, so the number of parts is raised beyond what fills the machine; keys near the start, in
    the middle and at the end are made to match the query."""
    n = 33000
    planted = [(0, 37), (0, 16511), (0, n - 2)]
    s = long_request(H, K, d, P, n, 1, seed=P + H, planted=planted[:1] if d == 64 else planted[1:2])
    scale = 1.0 / math.sqrt(d)
    width = s["bt"].shape[1]
    assert width > 2000
    splits = ops().decode_splits(1, K, H // K, n, width)
    assert splits >= (width + 1999) // 2000
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    want = long_reference(s, H, K, scale)
    for sp in sorted({splits, min(splits + 3, 64), 64}):
        out = torch.full_like(s["q"], float("nan"))
        dec = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops().paged_attention_decode(s["q"], s["k_pages"], s["v_pages"], dec, s["positions"], s["token_req"], s["bt"],
                                     scale, 0, sp, e, out)
        torch.cuda.synchronize()
        assert int(e.item()) == 0 and not torch.isnan(out).any()
        assert (out.double() - want).abs().max() <= 2e-2, (sp, float((out.double() - want).abs().max()))
    far = (planted[:1] if d == 64 else planted[1:2])[0][1]
    assert (out[0, 0].float() - s["vs"][far, 0].float()).abs().max() < 0.25       # dominated by the far key's value
    # fewer parts than the block table's width allows are refused, not run on a part of the table
    from ai_engine_b200.kernels.loader import KernelError
    if (width + 1) // 2 + 2 > 2048:
        with pytest.raises(KernelError):
            ops().paged_attention_decode(s["q"], s["k_pages"], s["v_pages"], dec, s["positions"], s["token_req"], s["bt"],
                                         scale, 0, 2, e, torch.empty_like(s["q"]))


@pytest.mark.parametrize("d,P", [(128, 16), (64, 8)])
def test_prompt_attention_2048_tokens_after_30720(d, P):
    """A portion of 2,048 prompt tokens whose request holds 30,720 tokens already: every CTA of the tcgen05
    kernel walks 241 to 256 key tiles, page ids read a tile ahead; rows at the start, in the middle and at the
    end of the portion each have a far key made for them (near the start, in the middle, just before the row)."""
    H, K = 4, 2
    n, n_q = 32768, 2048
    planted = [(0, 5), (1000, 10000), (2047, n - 3), (130, 30719)]
    s = long_request(H, K, d, P, n, n_q, seed=d + P, planted=planted)
    scale = 1.0 / math.sqrt(d)
    i32 = lambda a: torch.tensor(a, device=DEV, dtype=torch.int32)
    tiles = i32([[0, o] for o in range(0, n_q, ops().PREFILL_TILE)])
    e = torch.zeros(1, dtype=torch.int32, device=DEV)
    want = long_reference(s, H, K, scale)
    outs = {}
    units = i32([[0, o] for o in range(0, n_q, 2 * ops().PREFILL_TILE)])
    for name in ("tcgen05", "tcgen05_two_tiles", "mma_sync"):
        out = torch.full_like(s["q"], float("nan"))
        args = (s["q"], s["k_pages"], s["v_pages"], tiles, i32([0]), i32([n_q]), i32([n - n_q]), s["bt"], scale, 0, e, out)
        if name == "tcgen05":
            assert ops().paged_attention_prefill_tc(*args)
        elif name == "tcgen05_two_tiles":
            assert ops().paged_attention_prefill_tc(*args[:3], units, *args[4:], pair=True)
        else:
            ops().paged_attention_prefill(*args)
        torch.cuda.synchronize()
        assert int(e.item()) == 0 and not torch.isnan(out).any(), name
        err = (out.double() - want).abs().amax(dim=(1, 2))
        assert err.max() <= 2e-2, f"{name}: first wrong row {int((err > 2e-2).nonzero()[0])} of {n_q}: {float(err.max())}"
        outs[name] = out
    for row, far in planted:
        for name in ("tcgen05", "tcgen05_two_tiles"):
            assert (outs[name][row, 0].float() - s["vs"][far, 0].float()).abs().max() < 0.25, (name, row, far)
