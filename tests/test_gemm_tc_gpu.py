"""The tcgen05 / TMA matrix product alone against float64, over token counts from 1 to
thousands, widths that are no multiple of the tile, K with a ragged last block, every
token tile, and split K."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def run(T, N, K, out_dtype=torch.float32, bn=None, splits=None, seed=0):
    from ai_engine_b200.kernels import ops

    torch.manual_seed(seed)
    x = torch.randn(T, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = ops.gemm_tc(x, w, out_dtype, err, bn=bn, splits=splits)
    torch.cuda.synchronize()
    assert int(err.item()) == 0, "a bounded wait ran out"
    want = x.double() @ w.double().T
    tol = (2e-5 if out_dtype == torch.float32 else 1e-2) * max(1.0, float(want.abs().max())) * max(1.0, (K / 4096) ** 0.5)
    bad = (out.double() - want).abs()
    assert bad.max() <= tol, (T, N, K, bn, splits, float(bad.max()), tol, [int(i) for i in (bad > tol).nonzero()[0]])
    return out


def test_one_tile_one_block():
    run(16, 128, 64, bn=16, splits=1)


@pytest.mark.parametrize("T,N,K", [(8, 128, 64), (1, 256, 128), (16, 384, 512), (8, 4096, 4096), (8, 6144, 4096),
                                   (3, 100, 200), (5, 1000, 72), (16, 128256, 256), (8, 4096, 14336)])
def test_few_tokens(T, N, K):
    run(T, N, K)
    run(T, N, K, torch.bfloat16)


@pytest.mark.parametrize("bn", [16, 32, 64, 128, 256])
def test_every_token_tile(bn):
    run(bn, 512, 1024, bn=bn, splits=1)
    run(bn + 7, 300, 328, bn=bn, splits=1, seed=1)      # two token tiles, ragged N and K


@pytest.mark.parametrize("splits", [1, 2, 3, 7, 8])
def test_split_k(splits):
    run(8, 256, 2048, splits=splits)
    run(40, 200, 1032, bn=64, splits=splits, out_dtype=torch.bfloat16)


@pytest.mark.parametrize("T,N,K", [(300, 4096, 4096), (2048, 6144, 4096), (1000, 4096, 14336), (2048, 28672, 4096)])
def test_many_tokens(T, N, K):
    run(T, N, K, torch.bfloat16)


def test_a_token_does_not_depend_on_the_batch():
    from ai_engine_b200.kernels import ops

    torch.manual_seed(3)
    x = torch.randn(16, 4096, device=DEV).bfloat16()
    w = (torch.randn(512, 4096, device=DEV) * 0.05).bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    full = ops.gemm_tc(x, w, torch.float32, err, bn=16, splits=4)
    one = ops.gemm_tc(x[5:6].contiguous(), w, torch.float32, err, bn=16, splits=4)
    assert torch.equal(full[5], one[0])


@pytest.mark.parametrize("T,F,K,splits", [(8, 14336, 4096, 1), (1, 8192, 2048, 2), (16, 256, 192, 1), (40, 64, 64, 1),
                                          (12, 1024, 4096, 4), (64, 320, 4096, 8)])
def test_swiglu_epilogue_on_interleaved_tiles(T, F, K, splits):
    from ai_engine_b200.kernels import ops

    torch.manual_seed(F)
    x = torch.randn(T, K, device=DEV).bfloat16()
    g = (torch.randn(F, K, device=DEV) * 0.05).bfloat16()
    u = (torch.randn(F, K, device=DEV) * 0.05).bfloat16()
    w = torch.stack([g.view(-1, 64, K), u.view(-1, 64, K)], dim=1).reshape(2 * F, K).contiguous()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = ops.gemm_tc(x, w, torch.bfloat16, err, splits=splits, swiglu=True)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    gd, ud = x.double() @ g.double().T, x.double() @ u.double().T
    want = gd * torch.sigmoid(gd) * ud
    assert out.shape == (T, F)
    assert (out.double() - want).abs().max() <= 1e-2 * max(1.0, float(want.abs().max()))
    # the same through the part-level entry, and through the library product + interleaved activation
    a = ops.linear_swiglu(x, w, 64, err)
    b = ops.silu_mul(torch.mm(x, w.t()), block=64)
    assert (a.double() - want).abs().max() <= 1e-2 * max(1.0, float(want.abs().max()))
    assert (b.double() - want).abs().max() <= 1e-2 * max(1.0, float(want.abs().max()))


def test_linear_picks_the_kernel_by_step_size():
    from ai_engine_b200.kernels import ops

    torch.manual_seed(5)
    w = (torch.randn(384, 512, device=DEV) * 0.05).bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    for T in (1, 8, 64, 65, 300):
        x = torch.randn(T, 512, device=DEV).bfloat16()
        y = ops.linear(x, w, torch.float32, err)
        want = x.double() @ w.double().T
        assert y.dtype == torch.float32 and (y.double() - want).abs().max() <= 3e-5 * max(1.0, float(want.abs().max()))
    x = torch.randn(4, 100, device=DEV).bfloat16()          # K % 8 != 0: the library product stands in
    assert ops.linear(x, torch.randn(32, 100, device=DEV).bfloat16(), None, err).shape == (4, 32)


def test_raw_parts_are_summed_by_the_norm_and_rotary_kernels():
    """A split product may leave its parts unjoined: [parts, T, N] float32; the consumer adds them."""
    import plain_llama as pl
    from ai_engine_b200.kernels import ops

    torch.manual_seed(9)
    T, K, D = 8, 4096, 512
    x = torch.randn(T, K, device=DEV).bfloat16()
    w = (torch.randn(D, K, device=DEV) * 0.05).bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    parts = ops.gemm_tc(x, w, torch.float32, err, splits=4, raw_parts=True)
    assert parts.shape == (4, T, D) and parts.dtype == torch.float32
    want = x.double() @ w.double().T
    assert (parts.double().sum(0) - want).abs().max() <= 3e-5 * float(want.abs().max())
    resid = torch.randn(T, D, device=DEV)
    nw = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16()
    r2 = resid.clone()
    h = ops.add_rmsnorm(r2, parts, nw, 1e-5, torch.bfloat16)
    s = resid.double() + want
    assert (r2.double() - s).abs().max() <= 1e-4
    assert (h.double() - pl.rms_norm(s.cpu(), nw.double().cpu(), 1e-5).to(DEV)).abs().max() <= 3e-2
    assert int(err.item()) == 0


@pytest.mark.parametrize("T,N,K,splits", [(40, 6144, 4096, 9), (64, 256, 1024, 7), (1, 384, 640, 16), (8, 128, 64, 3),
                                          (33, 200, 4096, None), (64, 6144, 4096, None), (64, 3072, 8192, None),
                                          (17, 5120, 3072, None), (64, 2048, 2048, None)])
def test_unjoined_parts_cover_k_exactly(T, N, K, splits):
    """K blocks that do not divide into the asked number of parts (64 blocks in 9 parts): no part is left
    unwritten, whatever the output buffer held before (it is filled with NaN first)."""
    from ai_engine_b200.kernels import ops

    torch.manual_seed(T + N)
    x = torch.randn(T, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    poison = torch.full((32, T, N), float("nan"), device=DEV)      # the allocator hands this memory out next
    del poison
    parts = ops.gemm_tc(x, w, torch.float32, err, splits=splits, raw_parts=True) if splits else ops.linear_parts(x, w, err)
    assert bool(torch.isfinite(parts).all()), "a part of the output was not written"
    got = parts.sum(0) if parts.dim() == 3 else parts
    want = x.double() @ w.double().T
    assert (got.double() - want).abs().max() <= 3e-5 * max(1.0, float(want.abs().max())) * max(1.0, (K / 4096) ** 0.5)
    assert int(err.item()) == 0


@pytest.mark.parametrize("H,K,d,P,Kin,T", [(32, 8, 128, 16, 4096, 8), (32, 8, 64, 16, 2048, 3), (6, 1, 32, 8, 320, 16),
                                           (24, 8, 128, 32, 3072, 1), (4, 2, 16, 16, 64, 5)])
def test_qkv_product_with_rotation_and_cache_write_in_its_epilogue(H, K, d, P, Kin, T):
    """q/k/v product, rotation and page write in one kernel against the plain formulas: q rows, the rotated
    key and the value in the right slot of the right page, nothing else in the pool touched."""
    import plain_llama as pl
    from ai_engine_b200.kernels import ops

    torch.manual_seed(H + d + T)
    N = (H + 2 * K) * d
    x = torch.randn(T, Kin, device=DEV).bfloat16()
    w = (torch.randn(N, Kin, device=DEV) * (1.0 / Kin ** 0.5)).bfloat16()
    R, pages_per = 3, 6
    num_pages = R * pages_per + 2
    bt = torch.randperm(num_pages, device=DEV)[:R * pages_per].int().view(R, pages_per).contiguous()
    token_req = torch.tensor([t % R for t in range(T)], dtype=torch.int32, device=DEV)
    positions = torch.tensor([(7 * t + 3) % (pages_per * P) for t in range(T)], dtype=torch.int32, device=DEV)
    # two tokens of one request must not share a position
    seen = set()
    for t in range(T):
        while (int(token_req[t]), int(positions[t])) in seen:
            positions[t] = (int(positions[t]) + 1) % (pages_per * P)
        seen.add((int(token_req[t]), int(positions[t])))
    inv_freq = torch.from_numpy(pl.inv_freq_default(d, 500000.0)).to(DEV)
    kp = torch.full((num_pages, K, P, d), float("nan"), device=DEV, dtype=torch.bfloat16)
    vp = torch.full_like(kp, float("nan"))
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    q = ops.linear_rope_kv(x, w, kp, vp, positions, token_req, bt, inv_freq, H, K, d, err)
    assert q is not None and q.shape == (T, H, d)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    y = (x.double() @ w.double().T).view(T, H + 2 * K, d).cpu()
    pos = positions.cpu()
    rot = lambda t: pl.rope(t.transpose(0, 1), pos, pl.inv_freq_default(d, 500000.0)).transpose(0, 1)
    tol = 2e-2 * max(1.0, float(y.abs().max()))
    assert (q.double().cpu() - rot(y[:, :H])).abs().max() <= tol
    kr, vr = rot(y[:, H:H + K]), y[:, H + K:]
    touched = torch.zeros(kp.shape, dtype=torch.bool, device=DEV)
    for t in range(T):
        pg, sl = int(bt[int(token_req[t]), int(pos[t]) // P]), int(pos[t]) % P
        assert (kp[pg, :, sl].double().cpu() - kr[t]).abs().max() <= tol
        assert (vp[pg, :, sl].double().cpu() - vr[t]).abs().max() <= tol
        touched[pg, :, sl] = True
    assert bool(torch.isnan(kp[~touched]).all()) and bool(torch.isnan(vp[~touched]).all())
    # against the two-kernel path (same sums, same rotation): equal up to the order of the float32 adds
    kp2, vp2 = torch.zeros_like(kp), torch.zeros_like(vp)
    q2 = ops.rope_kv_write(ops.linear_parts(x, w, err), kp2, vp2, positions, token_req, bt, inv_freq, H, K, d, err)
    assert (q.float() - q2.float()).abs().max() <= tol / 4
    # write=False leaves the pool alone and still returns q
    kp3 = torch.full_like(kp, float("nan"))
    q3 = ops.linear_rope_kv(x, w, kp3, torch.full_like(kp, float("nan")), positions, token_req, bt, inv_freq, H, K, d,
                            err, write=False)
    assert torch.equal(q3, q) and bool(torch.isnan(kp3).all())
    # a block-table entry outside the pool is flagged, not followed
    bad = bt.clone()
    bad[int(token_req[0]), int(pos[0]) // P] = num_pages + 5
    ops.linear_rope_kv(x, w, torch.zeros_like(kp), torch.zeros_like(kp), positions, token_req, bad, inv_freq, H, K, d, err)
    torch.cuda.synchronize()
    assert int(err.item()) & 2
    err.zero_()
    # sizes it does not take
    assert ops.linear_rope_kv(torch.randn(17, Kin, device=DEV).bfloat16(), w, kp, vp, positions, token_req, bt, inv_freq,
                              H, K, d, err) is None


def test_a_bounded_wait_gives_up_and_the_step_runner_reports_it():
    """A barrier that nothing arrives at: the wait runs out after its limit, the kernel sets the
    device error word and returns; the context stays usable and check_errors raises."""
    from ctypes import c_int, c_void_p

    from ai_engine_b200.engine.step import StepError, StepRunner
    from ai_engine_b200.kernels.loader import library

    class _Model:
        device = torch.device(DEV)
        dtype = torch.float32

        def has_host_parts(self):
            return False

    runner = StepRunner(_Model(), cache=None)
    lib = library("gemm_tc.cu")
    assert lib.aie_tc_wait_selftest(c_void_p(runner.err.data_ptr()), c_int(2000),
                                    c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    torch.cuda.synchronize()
    assert int(runner.err.item()) & 4
    with pytest.raises(StepError, match="bounded wait"):
        runner.check_errors()
    runner.check_errors()                       # the word was cleared
    run(8, 256, 512)                            # and the device still works
