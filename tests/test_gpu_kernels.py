"""Each CUDA kernel alone against a plain float32 PyTorch reference of the same
operation, at sizes other than the engine's."""

import math

import pytest
import torch

import plain_llama

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def k():
    from inf_engine_b200 import kernels
    return kernels


def tol(dtype):
    return dict(atol=2e-6, rtol=1e-5) if dtype is torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("table_dtype", DTYPES)
def test_embed_gather(table_dtype):
    torch.manual_seed(0)
    table = torch.randn(301, 200, device=DEV).to(table_dtype)
    ids = torch.randint(0, 301, (37,), device=DEV, dtype=torch.int32)
    out = torch.empty(37, 200, device=DEV)
    k().embed_gather(ids, table, out)
    assert torch.equal(out, table.float()[ids.long()])


@pytest.mark.parametrize("act", DTYPES)
@pytest.mark.parametrize("gain_dtype", DTYPES)
@pytest.mark.parametrize("d", [48, 300, 2050])
def test_rmsnorm_with_residual_sum(act, gain_dtype, d):
    torch.manual_seed(1)
    n, eps = 19, 3e-6
    res = torch.randn(n, d, device=DEV) * 3
    delta = (torch.randn(n, d, device=DEV)).to(act)
    gain = (1 + 0.1 * torch.randn(d, device=DEV)).to(gain_dtype)
    ref_sum = res + delta.float()
    ref = plain_llama.rms_norm(ref_sum.cpu(), gain.float().cpu(), eps)
    out = torch.empty(n, d, device=DEV, dtype=act)
    r = res.clone()
    k().rmsnorm(r, delta, gain, out, eps)
    assert torch.allclose(r, ref_sum, atol=0, rtol=0)                  # the residual took the sum, in float32
    assert torch.allclose(out.float().cpu(), ref, **tol(act))
    # without a delta, and on gathered rows (the residual is left alone)
    r2 = res.clone()
    rows = torch.tensor([5, 0, 18], device=DEV, dtype=torch.int32)
    out2 = torch.empty(3, d, device=DEV, dtype=act)
    k().rmsnorm(r2, delta, gain, out2, eps, row_index=rows)
    assert torch.equal(r2, res)
    assert torch.allclose(out2.float().cpu(), ref[rows.long().cpu()], **tol(act))
    out3 = torch.empty(n, d, device=DEV, dtype=act)
    k().rmsnorm(r2, None, gain, out3, eps)
    assert torch.allclose(out3.float().cpu(), plain_llama.rms_norm(res.cpu(), gain.float().cpu(), eps), **tol(act))


@pytest.mark.parametrize("act", DTYPES)
def test_rope_and_cache_write(act):
    torch.manual_seed(2)
    n, H, Hk, hd, ps, n_pages = 23, 3, 1, 48, 8, 9
    cfgd = dict(head_dim=hd, hidden_size=H * hd, num_attention_heads=H, rope_theta=20000.0)
    cos_full, sin_full = plain_llama.rope_tables(cfgd, 500)
    cos, sin = cos_full[:, :hd // 2].contiguous().to(DEV), sin_full[:, :hd // 2].contiguous().to(DEV)
    qkv = torch.randn(n, (H + 2 * Hk) * hd, device=DEV).to(act)
    positions = torch.randint(0, 500, (n,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(ps * n_pages, device=DEV)[:n].to(torch.int32)
    slots[3] = -1                                                       # a padding token writes nothing
    kpool = torch.full((n_pages, Hk, ps, hd), 7.0, device=DEV, dtype=act)
    vpool = torch.full((n_pages, Hk, ps, hd), 7.0, device=DEV, dtype=act)
    q0 = qkv[:, :H * hd].float().cpu().view(n, H, hd)
    k0 = qkv[:, H * hd:(H + Hk) * hd].float().cpu().view(n, Hk, hd)
    v0 = qkv[:, (H + Hk) * hd:].float().cpu().view(n, Hk, hd)
    pos = positions.long().cpu()
    q_ref = torch.stack([plain_llama.apply_rope(q0[i][:, None], cos_full[pos[i]][None], sin_full[pos[i]][None])[:, 0] for i in range(n)])
    k_ref = torch.stack([plain_llama.apply_rope(k0[i][:, None], cos_full[pos[i]][None], sin_full[pos[i]][None])[:, 0] for i in range(n)])
    q, kk, v = qkv[:, :H * hd], qkv[:, H * hd:(H + Hk) * hd], qkv[:, (H + Hk) * hd:]
    k().rope_kv_write(q, kk, v, cos, sin, positions, slots, kpool, vpool, H, Hk, hd, ps)
    assert torch.allclose(q.float().cpu().view(n, H, hd), q_ref, **tol(act))
    written = torch.zeros(n_pages, ps, dtype=torch.bool)
    for i in range(n):
        s = int(slots[i])
        if s < 0:
            continue
        page, off = divmod(s, ps)
        written[page, off] = True
        assert torch.allclose(kpool[page, :, off].float().cpu(), k_ref[i], **tol(act))
        assert torch.equal(vpool[page, :, off].float().cpu(), v0[i])
    untouched = kpool.float().cpu()[~written[:, None, :].expand(n_pages, Hk, ps)]
    assert (untouched == 7.0).all()


@pytest.mark.parametrize("act", DTYPES)
def test_silu_mul(act):
    torch.manual_seed(3)
    n, inter = 13, 328
    gu = (torch.randn(n, 2 * inter, device=DEV) * 3).to(act)
    out = torch.empty(n, inter, device=DEV, dtype=act)
    k().silu_mul(gu, out)
    g, u = gu.float().cpu()[:, :inter], gu.float().cpu()[:, inter:]
    assert torch.allclose(out.float().cpu(), plain_llama.silu(g) * u, **tol(act))
    k().silu_mul(gu, out, interleaved=True)
    g, u = gu.float().cpu()[:, 0::2], gu.float().cpu()[:, 1::2]
    assert torch.allclose(out.float().cpu(), plain_llama.silu(g) * u, **tol(act))


@pytest.mark.parametrize("a_dt,w_dt,c_dt", [(torch.float32,) * 3, (torch.float32, torch.bfloat16, torch.float32),
                                            (torch.bfloat16, torch.float32, torch.bfloat16),
                                            (torch.bfloat16, torch.bfloat16, torch.float32),
                                            (torch.bfloat16, torch.bfloat16, torch.bfloat16)])
def test_gemm_simt_is_float32_and_batch_invariant(a_dt, w_dt, c_dt):
    torch.manual_seed(4)
    M, N, K = 37, 101, 77
    a = torch.randn(M, K, device=DEV).to(a_dt)
    w = torch.randn(N, K, device=DEV).to(w_dt)
    out = torch.empty(M, N, device=DEV, dtype=c_dt)
    k().gemm_simt(a, w, out)
    ref = (a.double().cpu() @ w.double().cpu().T).float()
    assert torch.allclose(out.float().cpu(), ref, **(dict(atol=1e-4, rtol=1e-5) if c_dt is torch.float32 else tol(c_dt)))
    one = torch.empty(1, N, device=DEV, dtype=c_dt)
    k().gemm_simt(a[5:6], w, one)
    assert torch.equal(one[0], out[5])                                   # a row does not depend on its neighbours
    # strided output (a column slice of a wider buffer)
    wide = torch.zeros(M, N + 11, device=DEV, dtype=c_dt)
    k().gemm_simt(a, w, wide[:, 11:])
    assert torch.equal(wide[:, 11:], out) and float(wide[:, :11].abs().sum()) == 0


@pytest.mark.parametrize("M", [1, 8, 13, 16, 17, 40, 64])
@pytest.mark.parametrize("N,K", [(389, 120), (96, 328), (2056, 512)])
def test_gemm_stream_plain_and_fused(M, N, K):
    torch.manual_seed(M * 1000 + N)
    bf = torch.bfloat16
    a = torch.randn(M, K, device=DEV).to(bf)
    w = (torch.randn(N, K, device=DEV) * 0.1).to(bf)
    ref = a.float().cpu() @ w.float().cpu().T
    scale = float(ref.abs().max())
    for nt in (1, 2, 4):
        if M > 32 and nt == 4:
            continue
        out = torch.full((M, N), float("nan"), device=DEV, dtype=bf)
        k().gemm_stream(a, w, out, M, "bf16", nt=nt)
        assert float((out.float().cpu() - ref).abs().max()) <= 1e-2 * scale
        out32 = torch.full((M, N), float("nan"), device=DEV)
        k().gemm_stream(a, w, out32, M, "f32", nt=nt)
        assert float((out32.cpu() - ref).abs().max()) <= 1e-4 * scale + 1e-5
    # residual epilogue: float32 accumulate in place
    res = torch.randn(M, N, device=DEV)
    want = res.cpu() + ref
    k().gemm_stream(a, w, res, M, "residual")
    assert float((res.cpu() - want).abs().max()) <= 1e-4 * scale + 1e-5
    # fused RMSNorm prologue on the float32 residual stream, rows gathered
    x = torch.randn(M + 5, K, device=DEV) * 2
    rows = torch.randperm(M + 5)[:M].to(torch.int32).to(DEV)
    for gain_dtype in (bf, torch.float32):
        gain = (1 + 0.1 * torch.randn(K, device=DEV)).to(gain_dtype)
        normed = plain_llama.rms_norm(x.cpu()[rows.long().cpu()], gain.float().cpu(), 1e-5)
        want = normed @ w.float().cpu().T
        out32 = torch.empty(M, N, device=DEV)
        k().gemm_stream(x, w, out32, M, "f32", gain=gain, eps=1e-5, row_index=rows)
        assert float((out32.cpu() - want).abs().max()) <= 1e-2 * float(want.abs().max())
    # silu(gate)*up over interleaved rows
    if N % 2 == 0:
        out = torch.empty(M, N // 2, device=DEV, dtype=bf)
        k().gemm_stream(a, w, out, M, "silu_mul")
        want = plain_llama.silu(ref[:, 0::2]) * ref[:, 1::2]
        assert float((out.float().cpu() - want).abs().max()) <= 1e-2 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(389, 256), (1000, 768), (2050, 2048), (776, 3072), (520, 8192)])
def test_gemm_stream_bulk_copy_kernel(M, N, K):
    """The persistent kernel (weights by cp.async.bulk through a shared-memory ring), default for K % 256 == 0."""
    from inf_engine_b200 import kernels
    lib = kernels.stream_library()
    assert lib.ie_gemm_stream_tma_supports(M, N, K, 0)
    torch.manual_seed(M * 7 + N)
    bf = torch.bfloat16
    a = torch.randn(M, K, device=DEV).to(bf)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(bf)
    ref = a.float().cpu() @ w.float().cpu().T
    scale = float(ref.abs().max())
    out32 = torch.full((M, N), float("nan"), device=DEV)
    k().gemm_stream(a, w, out32, M, "f32")
    assert float((out32.cpu() - ref).abs().max()) <= 2e-4 * scale + 1e-5
    old = torch.empty(M, N, device=DEV)
    k().gemm_stream(a, w, old, M, "f32", nt=1)                      # the register-streaming kernel agrees
    assert float((out32 - old).abs().max()) <= 2e-4 * scale + 1e-5
    out = torch.full((M, N), float("nan"), device=DEV, dtype=bf)
    k().gemm_stream(a, w, out, M, "bf16")
    assert float((out.float().cpu() - ref).abs().max()) <= 1e-2 * scale
    res = torch.randn(M, N, device=DEV)
    want = res.cpu() + ref
    k().gemm_stream(a, w, res, M, "residual")
    assert float((res.cpu() - want).abs().max()) <= 2e-4 * scale + 1e-5
    if lib.ie_gemm_stream_tma_supports(M, N, K, 1):
        x = torch.randn(M + 3, K, device=DEV) * 2
        rows = torch.randperm(M + 3)[:M].to(torch.int32).to(DEV)
        for gain_dtype in (bf, torch.float32):
            gain = (1 + 0.1 * torch.randn(K, device=DEV)).to(gain_dtype)
            normed = plain_llama.rms_norm(x.cpu()[rows.long().cpu()], gain.float().cpu(), 1e-5)
            want = normed @ w.float().cpu().T
            got = torch.empty(M, N, device=DEV)
            k().gemm_stream(x, w, got, M, "f32", gain=gain, eps=1e-5, row_index=rows)
            assert float((got.cpu() - want).abs().max()) <= 1e-2 * float(want.abs().max())
    if N % 2 == 0:
        h = torch.empty(M, N // 2, device=DEV, dtype=bf)
        k().gemm_stream(a, w, h, M, "silu_mul")
        want = plain_llama.silu(ref[:, 0::2]) * ref[:, 1::2]
        assert float((h.float().cpu() - want).abs().max()) <= 1e-2 * max(1.0, float(want.abs().max()))
    torch.cuda.synchronize()
    assert kernels.stream_error() == 0


@pytest.mark.parametrize("M,hidden,inter", [(8, 2048, 8192), (3, 1024, 2048), (13, 512, 1024), (16, 3072, 1024)])
def test_norm_handed_over_between_streaming_products(M, hidden, inter):
    """residual += h W_down^T with the next norm's input prepared on the way (bfloat16(residual * gain) and per-block
    sums of squares), then a product that takes that input instead of normalising the residual itself: both against
    float32 arithmetic, and the second against the same product with the RMSNorm prologue."""
    from inf_engine_b200 import kernels
    torch.manual_seed(hidden + M)
    bf = torch.bfloat16
    res0 = torch.randn(M, hidden, device=DEV)
    hmid = torch.randn(M, inter, device=DEV).to(bf)
    wd = (torch.randn(hidden, inter, device=DEV) * 0.03).to(bf)
    wq = (torch.randn(3 * 256, hidden, device=DEV) * 0.03).to(bf)
    eps = 1e-5
    for gain_dtype in (bf, torch.float32):
        gain = (1 + 0.1 * torch.randn(hidden, device=DEV)).to(gain_dtype)
        res = res0.clone()
        xg = torch.full((M, hidden), float("nan"), device=DEV, dtype=bf)
        ssq = torch.full((kernels.SSQ_SLOT, kernels.sm_count()), float("nan"), device=DEV)
        kernels.gemm_stream(hmid, wd, res, M, "residual", normout=(xg, gain, ssq))
        want_res = res0.cpu() + hmid.float().cpu() @ wd.float().cpu().T
        assert float((res.cpu() - want_res).abs().max()) <= 2e-3 * max(1.0, float(want_res.abs().max()))
        # what was prepared: bfloat16(residual * gain), and sums of squares that add up to the rows' own
        assert torch.equal(xg.float().cpu(), (res.cpu() * gain.float().cpu()).to(bf).float())
        total = ssq[:M].sum(dim=1).cpu()
        assert torch.allclose(total, (res.cpu() ** 2).sum(dim=1), rtol=1e-5)
        assert torch.isfinite(ssq).all() and (M == kernels.SSQ_SLOT or float(ssq[M:].abs().max()) == 0.0)
        # the product that takes it, against the one that normalises for itself
        out_a = torch.empty(M, wq.shape[0], device=DEV, dtype=bf)
        out_b = torch.empty_like(out_a)
        kernels.gemm_stream(xg, wq, out_a, M, "bf16", eps=eps, prenormed=(xg, ssq))
        kernels.gemm_stream(res, wq, out_b, M, "bf16", gain, eps)
        ref = plain_llama.rms_norm(res.cpu(), gain.float().cpu(), eps) @ wq.float().cpu().T
        scale = max(1.0, float(ref.abs().max()))
        assert float((out_a.float().cpu() - ref).abs().max()) <= 2e-2 * scale
        assert float((out_a.float() - out_b.float()).abs().max()) <= 1.6e-2 * scale      # a bfloat16 step of the result at most
    torch.cuda.synchronize()
    assert kernels.stream_error() == 0


def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable(monkeypatch):
    """The kernels that wait on barriers bound every wait and report a wait that ran out through an error word.
    A variant of the streaming product is compiled with a short limit and with every stage's barrier armed for 16
    bytes more than are copied: no stage ever completes, so the consumers and the producer each run into their
    limit, record it and leave.  Nothing faults and nothing hangs: the launch returns, the word is set,
    ``check_device_errors`` raises, and the next ordinary launch gives the right product."""
    from inf_engine_b200 import kernels
    from inf_engine_b200.kernels import KernelError
    torch.manual_seed(3)
    bf = torch.bfloat16
    M, N, K = 16, 256, 256
    a = torch.randn(M, K, device=DEV).to(bf)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(bf)
    ref = a.float().cpu() @ w.float().cpu().T
    assert kernels.stream_library().ie_gemm_stream_tma_supports(M, N, K, 0)
    stalled = kernels.stream_library({"IE_STREAM_SPIN_LIMIT": 512, "IE_STREAM_ARM_EXTRA": 16})
    assert stalled is not kernels.stream_library() and kernels.stream_error(stalled) == 0
    out = torch.zeros(M, N, device=DEV, dtype=bf)
    kernels.gemm_stream(a, w, out, M, "bf16", lib=stalled)
    torch.cuda.synchronize()                                     # the launch returns
    monkeypatch.setattr(kernels, "_stream_lib", stalled)         # let the engine's check look at this library
    with pytest.raises(KernelError, match="gave up a bounded wait"):
        kernels.check_device_errors()
    assert kernels.stream_error(stalled) == 0                    # reading clears the word
    monkeypatch.undo()
    good = torch.zeros(M, N, device=DEV, dtype=bf)
    kernels.gemm_stream(a, w, good, M, "bf16")
    torch.cuda.synchronize()
    assert kernels.stream_error() == 0
    assert float((good.float().cpu() - ref).abs().max()) <= 1e-2 * float(ref.abs().max())
    kernels.check_device_errors()


@pytest.mark.parametrize("M,N,K,bn", [(128, 256, 64, 256), (100, 200, 128, 128), (333, 1000, 512, 128),
                                      (700, 1306, 192, 256), (2048, 3072, 2048, 256), (520, 1024, 320, 256)])
def test_gemm_tcgen05_against_float32(M, N, K, bn):
    """TMA operands, tcgen05.mma with the accumulator in tensor memory, persistent over tiles, edge tiles included;
    tiles 128 and 256 wide.  Full tiles leave through shared memory, edge tiles straight from registers: the sizes
    have both."""
    torch.manual_seed(M + N)
    bf = torch.bfloat16
    a = torch.randn(M, K, device=DEV).to(bf)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(bf)
    ref = a.float().cpu() @ w.float().cpu().T
    scale = float(ref.abs().max())
    out = torch.full((M, N), float("nan"), device=DEV, dtype=bf)
    k().gemm_tcgen05(a, w, out, "bf16", bn)
    assert float((out.float().cpu() - ref).abs().max()) <= 1e-2 * scale
    res = torch.randn(M, N, device=DEV)
    want = res.cpu() + ref
    k().gemm_tcgen05(a, w, res, "residual", bn)
    assert float((res.cpu() - want).abs().max()) <= 2e-4 * scale + 1e-5
    h = torch.full((M, N // 2), float("nan"), device=DEV, dtype=bf)
    k().gemm_tcgen05(a, w, h, "silu_mul", bn)
    want = plain_llama.silu(ref[:, 0::2]) * ref[:, 1::2]
    assert float((h.float().cpu() - want).abs().max()) <= 1e-2 * max(1.0, float(want.abs().max()))
    torch.cuda.synchronize()
    assert k().gemm_tcgen05_error() == 0


def test_gemm_tcgen05_refuses_what_it_cannot_take():
    from inf_engine_b200.kernels import KernelError
    bf = torch.bfloat16
    assert not k().gemm_tcgen05_supports(128, 256, 120, 120, 120)      # K is no multiple of 64
    a, w = torch.zeros(4, 120, device=DEV, dtype=bf), torch.zeros(8, 120, device=DEV, dtype=bf)
    with pytest.raises(KernelError, match="size"):
        k().gemm_tcgen05(a, w, torch.zeros(4, 8, device=DEV, dtype=bf))


def test_gemm_stream_refuses_what_it_cannot_take():
    from inf_engine_b200.kernels import KernelError
    bf = torch.bfloat16
    a, w = torch.zeros(65, 64, device=DEV, dtype=bf), torch.zeros(8, 64, device=DEV, dtype=bf)
    with pytest.raises(KernelError, match="size"):
        k().gemm_stream(a, w, torch.zeros(65, 8, device=DEV, dtype=bf), 65)
    a, w = torch.zeros(4, 12, device=DEV, dtype=bf), torch.zeros(8, 12, device=DEV, dtype=bf)
    with pytest.raises(KernelError, match="size"):
        k().gemm_stream(a, w, torch.zeros(4, 8, device=DEV, dtype=bf), 4)


def paged_reference(q, kd, vd, q_lens, ctx_before, H, Hk, hd, window):
    """Dense float32 attention per request: q [N, H*hd]; kd/vd lists of [S_r, Hk, hd]."""
    outs = []
    g = H // Hk
    n0 = 0
    for r, ql in enumerate(q_lens):
        S = ctx_before[r] + ql
        kk = kd[r][:S].repeat_interleave(g, dim=1).transpose(0, 1)       # [H, S, hd]
        vv = vd[r][:S].repeat_interleave(g, dim=1).transpose(0, 1)
        qq = q[n0:n0 + ql].view(ql, H, hd).transpose(0, 1)               # [H, ql, hd]
        s = (qq @ kk.transpose(1, 2)) * hd ** -0.5
        i = torch.arange(ql)[:, None] + ctx_before[r]
        j = torch.arange(S)[None, :]
        ok = j <= i
        if window:
            ok &= j > i - window
        s = s.masked_fill(~ok[None], float("-inf"))
        outs.append((torch.softmax(s, -1) @ vv).transpose(0, 1).reshape(ql, H * hd))
        n0 += ql
    return torch.cat(outs)


def paged_case(act, H, Hk, hd, ps, q_lens, ctx_before, seed, spike=False):
    """Random requests laid out on shuffled pages; returns everything the kernels need."""
    g = torch.Generator().manual_seed(seed)
    R = len(q_lens)
    lens = [c + q for c, q in zip(ctx_before, q_lens)]
    n_pages_r = [-(-s // ps) for s in lens]
    n_pages = sum(n_pages_r) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(n_pages_r) + 2
    table = torch.full((R, width), -1, dtype=torch.int32)
    kpool = torch.full((n_pages, Hk, ps, hd), float("nan"))
    vpool = torch.full((n_pages, Hk, ps, hd), float("nan"))
    kd, vd = [], []
    for r in range(R):
        kr = torch.randn(lens[r], Hk, hd, generator=g)
        vr = torch.randn(lens[r], Hk, hd, generator=g)
        pages = [perm.pop() for _ in range(n_pages_r[r])]
        table[r, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        kd.append(kr)
        vd.append(vr)
    N = sum(q_lens)
    q = torch.randn(N, H * hd, generator=g)
    if spike:
        # one far key per request stands out for every query head: its score dominates the softmax
        n0 = 0
        for r in range(R):
            far = max(0, ctx_before[r] // 3)
            kd[r][far] = 0
            kd[r][far, :, 0] = 30.0
            q[n0:n0 + q_lens[r]].view(q_lens[r], H, hd)[:, :, 0] = 8.0
            n0 += q_lens[r]
    kd = [t.to(act).float() for t in kd]
    vd = [t.to(act).float() for t in vd]
    q = q.to(act).float()
    for r in range(R):
        for p, page in enumerate(table[r, :n_pages_r[r]].tolist()):
            n = min(ps, lens[r] - p * ps)
            kpool[page, :, :n] = kd[r][p * ps:p * ps + n].transpose(0, 1)
            vpool[page, :, :n] = vd[r][p * ps:p * ps + n].transpose(0, 1)
    # what lies beyond a request's length on its last page, and pages it does not own, stays NaN: poison that must
    # never reach an output (a kernel may load it, but only under a mask that replaces it, never under a weight of zero)
    q_start = [0]
    for ql in q_lens:
        q_start.append(q_start[-1] + ql)
    return dict(q=q, kd=kd, vd=vd, kpool=kpool, vpool=vpool, table=table, q_start=q_start, N=N, R=R)


def work_list(q_lens, group, rows):
    req, pair0 = [], []
    for r, ql in enumerate(q_lens):
        for p in range(0, ql * group, rows):
            req.append(r)
            pair0.append(p)
    return req, pair0


CASES = [
    # H, Hk, hd, page, q_lens, ctx_before, window
    (4, 2, 16, 16, [33], [0], None),
    (6, 2, 32, 8, [1, 9, 1, 40], [70, 0, 129, 31], None),
    (3, 1, 48, 8, [5, 1], [11, 200], None),
    (8, 8, 64, 16, [17, 1, 1], [0, 300, 15], None),
    (4, 1, 128, 16, [20, 1], [50, 333], None),
    (2, 1, 256, 4, [3, 1], [9, 40], None),
    (4, 2, 32, 8, [30, 1, 7], [0, 90, 41], 13),
    (5, 5, 80, 16, [2, 64], [62, 0], 33),
]


@pytest.mark.parametrize("act", DTYPES)
@pytest.mark.parametrize("case", CASES)
def test_attention_general(act, case):
    H, Hk, hd, ps, q_lens, ctx_before, window = case
    c = paged_case(act, H, Hk, hd, ps, q_lens, ctx_before, seed=hd + len(q_lens))
    ref = paged_reference(c["q"], c["kd"], c["vd"], q_lens, ctx_before, H, Hk, hd, window)
    req, pair0 = work_list(q_lens, H // Hk, 32)
    dev = lambda t, dt=torch.int32: torch.as_tensor(t, dtype=dt).to(DEV)
    out = torch.full((c["N"], H * hd), float("nan"), device=DEV, dtype=act)
    k().attention_general(c["q"].to(DEV, act), out, c["kpool"].to(DEV, act), c["vpool"].to(DEV, act),
                          c["table"].to(DEV), dev(c["q_start"]), dev(ctx_before), dev(req), dev(pair0), len(req),
                          H, Hk, hd, ps, window, hd ** -0.5)
    assert torch.allclose(out.float().cpu(), ref, **(dict(atol=1e-5, rtol=1e-5) if act is torch.float32 else tol(act)))


@pytest.mark.parametrize("act", DTYPES)
def test_attention_finds_one_far_key_among_hundreds(act):
    H, Hk, hd, ps = 4, 2, 32, 8
    q_lens, ctx_before = [1, 6], [700, 420]
    c = paged_case(act, H, Hk, hd, ps, q_lens, ctx_before, seed=11, spike=True)
    ref = paged_reference(c["q"], c["kd"], c["vd"], q_lens, ctx_before, H, Hk, hd, None)
    # the reference itself is, to rounding, the value stored at the far key
    far0 = c["vd"][0][700 // 3].repeat_interleave(2, dim=0).reshape(-1)
    assert torch.allclose(ref[0], far0, atol=1e-3)
    req, pair0 = work_list(q_lens, 2, 32)
    dev = lambda t: torch.as_tensor(t, dtype=torch.int32).to(DEV)
    out = torch.empty((c["N"], H * hd), device=DEV, dtype=act)
    k().attention_general(c["q"].to(DEV, act), out, c["kpool"].to(DEV, act), c["vpool"].to(DEV, act),
                          c["table"].to(DEV), dev(c["q_start"]), dev(ctx_before), dev(req), dev(pair0), len(req),
                          H, Hk, hd, ps, None, hd ** -0.5)
    assert torch.allclose(out.float().cpu(), ref, **(dict(atol=1e-5, rtol=1e-5) if act is torch.float32 else tol(act)))


MMA_CASES = [
    # H, Hk, hd, page, q_lens, ctx_before, window
    (8, 2, 64, 16, [200], [0], None),
    (6, 2, 64, 8, [1, 9, 1, 70, 130], [70, 0, 129, 31, 515], None),
    (4, 4, 64, 16, [17, 1, 64], [3, 300, 64], None),
    (3, 1, 64, 4, [5, 66], [11, 200], None),
    (4, 1, 128, 16, [20, 1, 100], [50, 333, 0], None),
    (2, 2, 128, 32, [3, 150], [9, 40], None),
    (8, 2, 64, 16, [30, 1, 7, 200], [0, 90, 41, 100], 37),
    (2, 1, 128, 8, [2, 64, 1], [62, 0, 500], 70),
]


@pytest.mark.parametrize("rows", [64, 128])
@pytest.mark.parametrize("case", MMA_CASES)
def test_attention_prefill_tensor_cores(case, rows):
    H, Hk, hd, ps, q_lens, ctx_before, window = case
    act = torch.bfloat16
    c = paged_case(act, H, Hk, hd, ps, q_lens, ctx_before, seed=3 * hd + len(q_lens))
    ref = paged_reference(c["q"], c["kd"], c["vd"], q_lens, ctx_before, H, Hk, hd, window)
    req, pair0 = work_list(q_lens, H // Hk, rows)
    dev = lambda t: torch.as_tensor(t, dtype=torch.int32).to(DEV)
    out = torch.full((c["N"], H * hd), float("nan"), device=DEV, dtype=act)
    k().attention_prefill_mma(c["q"].to(DEV, act), out, c["kpool"].to(DEV, act), c["vpool"].to(DEV, act),
                              c["table"].to(DEV), dev(c["q_start"]), dev(ctx_before), dev(req), dev(pair0), len(req),
                              H, Hk, hd, ps, window, hd ** -0.5, rows)
    assert torch.allclose(out.float().cpu(), ref, **tol(act))


TCGEN05_ATTENTION_CASES = [
    # H, Hk, hd, page, q_lens, ctx_before
    (8, 2, 64, 16, [200], [0]),
    (6, 2, 64, 8, [1, 9, 1, 70, 130], [70, 0, 129, 31, 515]),
    (4, 4, 64, 16, [17, 1, 64, 300], [3, 300, 64, 0]),
    (3, 1, 64, 32, [5, 166], [11, 200]),
    (8, 1, 64, 64, [129, 2], [127, 1000]),
    (2, 2, 64, 64, [3, 150, 257], [9, 40, 0]),
    (8, 2, 128, 16, [200], [0]),
    (6, 2, 128, 8, [1, 9, 1, 70, 130], [70, 0, 129, 31, 515]),
    (3, 3, 128, 32, [17, 1, 300], [3, 300, 64]),
    (4, 1, 128, 64, [129, 2, 40], [127, 1000, 0]),
    # long: the rings of stages and of S buffers go round many times
    (4, 2, 64, 16, [2500, 40], [0, 3000]),
    (2, 1, 128, 16, [1500], [1200]),
]


@pytest.mark.parametrize("case", TCGEN05_ATTENTION_CASES)
def test_attention_prefill_tcgen05(case):
    H, Hk, hd, ps, q_lens, ctx_before = case
    act = torch.bfloat16
    assert k().attention_tcgen05_supports(hd, ps, None)
    c = paged_case(act, H, Hk, hd, ps, q_lens, ctx_before, seed=5 * ps + len(q_lens) + hd)
    ref = paged_reference(c["q"], c["kd"], c["vd"], q_lens, ctx_before, H, Hk, hd, None)
    req, pair0 = work_list(q_lens, H // Hk, 128)
    dev = lambda t: torch.as_tensor(t, dtype=torch.int32).to(DEV)
    out = torch.full((c["N"], H * hd), float("nan"), device=DEV, dtype=act)
    k().attention_tcgen05(c["q"].to(DEV, act), out, c["kpool"].to(DEV, act), c["vpool"].to(DEV, act),
                          c["table"].to(DEV), dev(c["q_start"]), dev(ctx_before), dev(req), dev(pair0), len(req),
                          H, Hk, hd, ps, hd ** -0.5)
    torch.cuda.synchronize()
    assert k().attention_tcgen05_error() == 0
    assert torch.allclose(out.float().cpu(), ref, **tol(act))


@pytest.mark.parametrize("hd", [64, 128])
def test_attention_tcgen05_rotates_q_as_it_reads_it(hd):
    """q arrives unrotated with tables and positions; the result equals attention over q rotated on the host."""
    H, Hk, ps, act = 6, 2, 16, torch.bfloat16
    q_lens, ctx_before = [140, 50], [37, 300]
    c = paged_case(act, H, Hk, hd, ps, q_lens, ctx_before, seed=21 + hd)
    half = hd // 2
    g = torch.Generator().manual_seed(3)
    n_pos = max(a + b for a, b in zip(q_lens, ctx_before))
    ang = torch.rand(n_pos, half, generator=g) * 6.28
    cos, sin = ang.cos(), ang.sin()
    positions = [cb + i for ql, cb in zip(q_lens, ctx_before) for i in range(ql)]
    q_raw = c["q"]                                              # bfloat16-rounded values
    qr = q_raw.view(-1, H, hd)
    cc, ss = cos[positions][:, None, :], sin[positions][:, None, :]
    a, b = qr[..., :half], qr[..., half:]
    q_rot = torch.cat([a * cc - b * ss, b * cc + a * ss], dim=-1).to(act).float().view(-1, H * hd)
    ref = paged_reference(q_rot, c["kd"], c["vd"], q_lens, ctx_before, H, Hk, hd, None)
    req, pair0 = work_list(q_lens, H // Hk, 128)
    dev = lambda t: torch.as_tensor(t, dtype=torch.int32).to(DEV)
    out = torch.full((c["N"], H * hd), float("nan"), device=DEV, dtype=act)
    qd = q_raw.to(DEV, act)
    k().attention_tcgen05(qd, out, c["kpool"].to(DEV, act), c["vpool"].to(DEV, act), c["table"].to(DEV),
                          dev(c["q_start"]), dev(ctx_before), dev(req), dev(pair0), len(req), H, Hk, hd, ps, hd ** -0.5,
                          cos.to(DEV), sin.to(DEV), dev(positions))
    torch.cuda.synchronize()
    assert k().attention_tcgen05_error() == 0
    assert torch.allclose(out.float().cpu(), ref, **tol(act))
    assert torch.equal(qd.float().cpu(), q_raw)                 # q itself is left as it came


@pytest.mark.parametrize("hd", [64, 128])
def test_attention_tcgen05_finds_one_far_key_among_hundreds(hd):
    H, Hk, ps, act = 4, 2, 16, torch.bfloat16
    q_lens, ctx_before = [140, 6], [700, 420]
    c = paged_case(act, H, Hk, hd, ps, q_lens, ctx_before, seed=11, spike=True)
    ref = paged_reference(c["q"], c["kd"], c["vd"], q_lens, ctx_before, H, Hk, hd, None)
    req, pair0 = work_list(q_lens, 2, 128)
    dev = lambda t: torch.as_tensor(t, dtype=torch.int32).to(DEV)
    out = torch.empty((c["N"], H * hd), device=DEV, dtype=act)
    k().attention_tcgen05(c["q"].to(DEV, act), out, c["kpool"].to(DEV, act), c["vpool"].to(DEV, act),
                          c["table"].to(DEV), dev(c["q_start"]), dev(ctx_before), dev(req), dev(pair0), len(req),
                          H, Hk, hd, ps, hd ** -0.5)
    torch.cuda.synchronize()
    assert k().attention_tcgen05_error() == 0
    assert torch.allclose(out.float().cpu(), ref, **tol(act))


def test_attention_tcgen05_refuses_what_it_cannot_do():
    assert not k().attention_tcgen05_supports(96, 16, None)
    assert not k().attention_tcgen05_supports(128, 128, None)
    assert not k().attention_tcgen05_supports(64, 128, None)
    assert not k().attention_tcgen05_supports(64, 4, None)
    assert not k().attention_tcgen05_supports(64, 16, 32)


DECODE_CASES = [
    # H, Hk, hd, page, q_lens, ctx_before, window, split_keys
    (8, 2, 64, 16, [1, 1, 1], [0, 700, 33], None, 64),
    (32, 8, 64, 16, [1] * 5, [2047, 1, 511, 512, 100], None, 128),
    (6, 2, 64, 8, [2, 1, 5], [70, 0, 129], None, 32),
    (4, 4, 64, 16, [1, 16], [300, 15], None, 256),
    (4, 1, 128, 16, [1, 3], [333, 50], None, 96),
    (16, 1, 128, 32, [1], [900], None, 128),
    (8, 2, 64, 16, [1, 1, 2], [90, 41, 400], 37, 64),
    # long contexts: more blocks per stream than one round of the last block's merge takes
    (8, 2, 64, 16, [1, 1], [9000, 5], None, 64),
    (4, 1, 128, 16, [1, 2], [7, 6100], None, 64),
    # head size 128 walks the keys in tiles of 16: splits that are no multiple of a page, pages of 32, a group of 3
    (24, 8, 128, 32, [1, 1], [3000, 40], None, 96),
    # every size of the cluster that adds the blocks of a (request, kv head) up: 4 to 8 blocks of six warps for
    # the long request, while the short one's other blocks have no keys
    (8, 2, 64, 16, [1, 1], [1394, 5], None, 64),
    (8, 2, 64, 16, [1, 1], [1778, 900], None, 64),
    (8, 2, 64, 16, [1, 2], [2162, 5], None, 64),
    (8, 2, 64, 16, [1, 1], [2546, 5], None, 64),
    (8, 2, 64, 16, [1, 1], [2930, 2000], None, 64),
    (4, 1, 128, 16, [1, 1], [818, 3], None, 64),
    (4, 1, 128, 16, [1, 1], [1202, 3], None, 64),
    (4, 1, 128, 16, [2, 1], [1394, 700], None, 64),
]


@pytest.mark.parametrize("case", DECODE_CASES)
def test_attention_decode_split_keys(case):
    H, Hk, hd, ps, q_lens, ctx_before, window, split_keys = case
    act = torch.bfloat16
    assert max(q_lens) * (H // Hk) <= 16
    c = paged_case(act, H, Hk, hd, ps, q_lens, ctx_before, seed=5 * hd + len(q_lens))
    ref = paged_reference(c["q"], c["kd"], c["vd"], q_lens, ctx_before, H, Hk, hd, window)
    dev = lambda t: torch.as_tensor(t, dtype=torch.int32).to(DEV)
    cap = max(a + b for a, b in zip(q_lens, ctx_before)) + 77      # the cap may exceed every request's length
    n_splits = -(-cap // split_keys)
    n = k().attention_decode_scratch_floats(c["N"], H, n_splits, hd)
    scratch = torch.full((n,), float("nan"), device=DEV)            # whatever an earlier call left must not matter,
    scratch[:k().attention_decode_ticket_words(hd)] = 0              # except the tickets, which start at zero
    out = torch.full((c["N"], H * hd), float("nan"), device=DEV, dtype=act)
    for _ in range(2):
        k().attention_decode_mma(c["q"].to(DEV, act), out, c["kpool"].to(DEV, act), c["vpool"].to(DEV, act),
                                 c["table"].to(DEV), dev(c["q_start"]), dev(ctx_before), scratch, len(q_lens),
                                 c["N"], H, Hk, hd, ps, window, hd ** -0.5, n_splits, split_keys)
        assert torch.allclose(out.float().cpu(), ref, **tol(act))


FUSED_DECODE_CASES = [
    # H, Hk, hd, page, ctx_before, window, split_keys, rotate, write_kv
    (8, 2, 64, 16, [0, 300, 15, 511, 512], None, 64, True, True),
    (6, 2, 64, 8, [70, 129, 31], None, 128, True, True),
    (4, 1, 128, 16, [50, 333, 0, 127], None, 64, True, True),
    (4, 4, 64, 16, [3, 1000], 37, 256, True, True),
    (8, 2, 64, 16, [64, 200], None, 64, False, True),
    (8, 2, 64, 16, [64, 200], None, 64, True, False),
    (8, 2, 64, 16, [6000, 100], None, 64, True, True),
    (24, 8, 128, 16, [2100, 97, 15], None, 96, True, True),
]


@pytest.mark.parametrize("case", FUSED_DECODE_CASES)
def test_attention_decode_with_rotation_and_cache_write_folded_in(case):
    """One token per request: q and the new key arrive unrotated, the kernel rotates them, puts the new key and
    value among the keys of the step and stores them in the pool; compared with rotation in float32 on the
    host followed by plain attention, and with the pool the separate kernels would leave."""
    H, Hk, hd, ps, ctx_before, window, split_keys, rotate, write_kv = case
    act = torch.bfloat16
    R = len(ctx_before)
    q_lens = [1] * R
    c = paged_case(act, H, Hk, hd, ps, q_lens, ctx_before, seed=7 * hd + R)
    g = torch.Generator().manual_seed(R)
    half = hd // 2
    n_pos = max(ctx_before) + 1
    ang = torch.rand(n_pos, half, generator=g) * 6.28
    cos, sin = (ang.cos(), ang.sin()) if rotate else (None, None)

    def rot(x, pos):                               # x [heads, hd] float32
        if not rotate:
            return x
        a, b = x[:, :half], x[:, half:]
        cc, ss = cos[pos][None], sin[pos][None]
        return torch.cat([a * cc - b * ss, b * cc + a * ss], dim=1)

    # the step's own token: raw q / k / v as the projections give them (bfloat16 values)
    q_raw = c["q"]                                                       # [R, H*hd], already bfloat16-rounded
    k_raw = torch.stack([c["kd"][r][ctx_before[r]] for r in range(R)])   # [R, Hk, hd]
    v_raw = torch.stack([c["vd"][r][ctx_before[r]] for r in range(R)])
    q_rot = torch.stack([rot(q_raw[r].view(H, hd), ctx_before[r]) for r in range(R)]).to(act).float().view(R, H * hd)
    k_rot = torch.stack([rot(k_raw[r], ctx_before[r]) for r in range(R)]).to(act).float()
    kd = [t.clone() for t in c["kd"]]
    for r in range(R):
        kd[r][ctx_before[r]] = k_rot[r]
    ref = paged_reference(q_rot, kd, c["vd"], q_lens, ctx_before, H, Hk, hd, window)

    # pools: poison where the new token goes when the kernel is to write it, the rotated key when it is not
    kpool, vpool = c["kpool"].clone(), c["vpool"].clone()
    slots = []
    for r in range(R):
        page = int(c["table"][r, ctx_before[r] // ps])
        off = ctx_before[r] % ps
        slots.append(page * ps + off)
        kpool[page, :, off] = float("nan") if write_kv else k_rot[r]
        if write_kv:
            vpool[page, :, off] = float("nan")
    kpool, vpool = kpool.to(DEV, act), vpool.to(DEV, act)
    dev = lambda t: torch.as_tensor(t, dtype=torch.int32).to(DEV)
    qkv = torch.cat([q_raw, k_raw.reshape(R, Hk * hd), v_raw.reshape(R, Hk * hd)], dim=1).to(DEV, act)
    qw, kw = H * hd, Hk * hd
    cap = max(ctx_before) + 1 + 50
    n_splits = -(-cap // split_keys)
    scratch = torch.zeros(k().attention_decode_scratch_floats(R, H, n_splits, hd), device=DEV)
    out = torch.full((R, H * hd), float("nan"), device=DEV, dtype=act)
    k().attention_decode_fused(qkv[:, :qw], qkv[:, qw:qw + kw], qkv[:, qw + kw:], out, kpool, vpool,
                               c["table"].to(DEV), dev(c["q_start"]), dev(ctx_before), scratch,
                               cos.to(DEV) if rotate else None, sin.to(DEV) if rotate else None, dev(ctx_before),
                               dev(slots), R, H, Hk, hd, ps, window, hd ** -0.5, write_kv, n_splits, split_keys)
    assert torch.allclose(out.float().cpu(), ref, **tol(act))
    for r in range(R):
        page, off = slots[r] // ps, slots[r] % ps
        assert torch.allclose(kpool[page, :, off].float().cpu(), k_rot[r], atol=2e-2, rtol=2e-2)
        assert torch.equal(vpool[page, :, off].float().cpu(), v_raw[r])
    # the unrotated inputs are left as they were
    assert torch.equal(qkv[:, :qw].float().cpu(), q_raw)


@pytest.mark.parametrize("kind", ["prefill", "decode"])
def test_tensor_core_attention_finds_one_far_key_among_hundreds(kind):
    H, Hk, hd, ps, act = 4, 2, 64, 16, torch.bfloat16
    q_lens, ctx_before = ([1, 6], [700, 420]) if kind == "prefill" else ([1, 1], [700, 420])
    if kind == "prefill":
        q_lens = [1, 40]
    c = paged_case(act, H, Hk, hd, ps, q_lens, ctx_before, seed=12, spike=True)
    ref = paged_reference(c["q"], c["kd"], c["vd"], q_lens, ctx_before, H, Hk, hd, None)
    dev = lambda t: torch.as_tensor(t, dtype=torch.int32).to(DEV)
    out = torch.empty((c["N"], H * hd), device=DEV, dtype=act)
    args = (c["q"].to(DEV, act), out, c["kpool"].to(DEV, act), c["vpool"].to(DEV, act), c["table"].to(DEV),
            dev(c["q_start"]), dev(ctx_before))
    if kind == "prefill":
        req, pair0 = work_list(q_lens, 2, 64)
        k().attention_prefill_mma(*args, dev(req), dev(pair0), len(req), H, Hk, hd, ps, None, hd ** -0.5)
    else:
        n_splits = -(-701 // 64)
        scratch = torch.zeros(k().attention_decode_scratch_floats(c["N"], H, n_splits, hd), device=DEV)
        k().attention_decode_mma(*args, scratch, 2, c["N"], H, Hk, hd, ps, None, hd ** -0.5, n_splits, 64)
    assert torch.allclose(out.float().cpu(), ref, **tol(act))


def test_attention_refuses_head_sizes_it_cannot_take():
    from inf_engine_b200.kernels import KernelError
    z = torch.zeros(1, device=DEV)
    zi = torch.zeros(2, device=DEV, dtype=torch.int32)
    with pytest.raises(KernelError, match="size"):
        k().attention_general(z.view(1, 1), z.view(1, 1), z, z, zi.view(1, 2), zi, zi, zi, zi, 1, 1, 1, 24, 8, None, 1.0)


# ------------------------------------------------------------------------ sampling
def test_argmax_takes_the_first_maximum():
    torch.manual_seed(5)
    logits = torch.randn(9, 3001, device=DEV)
    logits[2, 77] = logits[2, 1500] = 50.0
    out = torch.empty(9, device=DEV, dtype=torch.int32)
    k().argmax(logits, out)
    ref = logits.cpu().argmax(-1)
    assert out.cpu().tolist() == ref.tolist() and out[2] == 77


def test_repetition_penalty():
    torch.manual_seed(6)
    logits = torch.randn(3, 500, device=DEV)
    ctx = torch.full((3, 256), -1, dtype=torch.int32)
    seen = [[4, 9, 4, 499, 0], [], [7] * 40]
    for i, s in enumerate(seen):
        ctx[i, :len(s)] = torch.tensor(s, dtype=torch.int32)
    pen = torch.tensor([1.3, 1.0, 2.0], device=DEV)
    ref = torch.stack([plain_llama.apply_repetition_penalty(logits[i].cpu(), seen[i], float(pen[i])) for i in range(3)])
    k().repetition_penalty(logits, ctx.to(DEV), pen)
    assert torch.allclose(logits.cpu(), ref, atol=1e-6)


def _rows(configs, keys, vocab):
    import numpy as np
    from inf_engine_b200.sampling import SamplingMode
    rows = np.zeros((len(configs), 7), dtype=np.int32)
    f, u = rows.view(np.float32), rows.view(np.uint32)
    for i, c in enumerate(configs):
        if c.mode is SamplingMode.GREEDY:
            f[i, 0], f[i, 1] = 0.0, 1.0
        else:
            f[i, 0] = c.temperature
            f[i, 1] = c.top_p if c.mode is SamplingMode.TOP_P else 1.0
            rows[i, 2] = max(1, min(c.top_k, vocab)) if c.mode is SamplingMode.TOP_K else 0
        u[i, 3], u[i, 4] = c.seed & 0xFFFFFFFF, c.seed >> 32
        u[i, 5], u[i, 6] = keys[i] & 0xFFFFFFFF, keys[i] >> 32
    return torch.from_numpy(rows).to(DEV)


@pytest.mark.parametrize("vocab", [389, 5003])
def test_sampling_follows_the_plain_distribution_and_the_hashed_uniform(vocab):
    from inf_engine_b200.sampling import SamplingConfig, uniform_of
    torch.manual_seed(7)
    modes = [("greedy", {}), ("temperature", dict(temperature=0.7)), ("top_k", dict(top_k=5, temperature=1.3)),
             ("top_p", dict(top_p=0.6, temperature=0.9)), ("top_p", dict(top_p=1.0)), ("top_k", dict(top_k=10 ** 6))]
    n_draws = 40
    configs, keys = [], []
    for mode, kw in modes:
        for d in range(n_draws):
            configs.append(SamplingConfig(mode=mode, seed=1234 + len(mode), **kw))
            keys.append((3 << 32) | d)
    logits = (torch.randn(len(modes), vocab) * 2.5)
    logits[2, 10] = logits[2, 20] = logits[2].topk(5).values[-1]        # a tie on the top-k edge: both stay
    big = logits.repeat_interleave(n_draws, dim=0).contiguous().to(DEV)
    out = torch.empty(big.shape[0], device=DEV, dtype=torch.int32)
    k().sample(big, _rows(configs, keys, vocab), out)
    out = out.cpu().tolist()
    for i, c in enumerate(configs):
        row = logits[i // n_draws]
        probs = plain_llama.filtered_distribution(row, c.mode.value, c.temperature, c.top_k, c.top_p).double()
        tok = out[i]
        assert probs[tok] > 0, f"{c.mode} drew token {tok} that the filter removed"
        if c.mode.value == "greedy":
            assert tok == int(row.argmax())
            continue
        cdf = probs.cumsum(0)
        u = uniform_of(c.seed, keys[i])
        lo = float(cdf[tok - 1]) if tok > 0 else 0.0
        assert lo - 1e-5 <= u <= float(cdf[tok]) + 1e-5, f"{c.mode}: u={u} outside [{lo}, {float(cdf[tok])}] of token {tok}"
    # the draws of one row spread over several tokens (the hash differs with the key)
    assert len(set(out[n_draws:2 * n_draws])) >= 2


def test_greedy_rows_of_a_large_vocabulary_beside_sampled_rows():
    """Above 32,768 entries greedy rows are answered by 64 blocks a row; the other rows by the sampling kernel."""
    from inf_engine_b200.sampling import SamplingConfig, uniform_of
    torch.manual_seed(9)
    vocab = 40003
    logits = torch.randn(6, vocab) * 2
    logits[1, 30000] = logits[1, 123] = 60.0                        # a tie across two slices: the lower index wins
    logits[3, vocab - 1] = 70.0                                      # the very last entry
    cfgs = [SamplingConfig(), SamplingConfig(), SamplingConfig(mode="temperature", temperature=0.8, seed=3),
            SamplingConfig(), SamplingConfig(mode="top_k", top_k=4, seed=3), SamplingConfig()]
    keys = [(i << 32) | 1 for i in range(6)]
    out = torch.full((6,), -1, device=DEV, dtype=torch.int32)
    for _ in range(2):                                               # the tickets go back to zero after a launch
        k().sample(logits.to(DEV), _rows(cfgs, keys, vocab), out)
        got = out.cpu().tolist()
        for i in (0, 1, 3, 5):
            assert got[i] == int(logits[i].argmax()), i
        assert got[1] == 123 and got[3] == vocab - 1
        for i in (2, 4):
            probs = plain_llama.filtered_distribution(logits[i], cfgs[i].mode.value, cfgs[i].temperature, cfgs[i].top_k, 1.0).double()
            cdf = probs.cumsum(0)
            u = uniform_of(cfgs[i].seed, keys[i])
            lo = float(cdf[got[i] - 1]) if got[i] > 0 else 0.0
            assert probs[got[i]] > 0 and lo - 1e-5 <= u <= float(cdf[got[i]]) + 1e-5


def test_sampling_is_reproducible_and_independent_of_the_batch():
    from inf_engine_b200.sampling import SamplingConfig
    torch.manual_seed(8)
    logits = torch.randn(6, 1000, device=DEV)
    cfgs = [SamplingConfig(mode="top_p", top_p=0.8, temperature=1.1, seed=5) for _ in range(6)]
    keys = [(i << 32) | 4 for i in range(6)]
    a = torch.empty(6, device=DEV, dtype=torch.int32)
    b = torch.empty(6, device=DEV, dtype=torch.int32)
    k().sample(logits, _rows(cfgs, keys, 1000), a)
    k().sample(logits, _rows(cfgs, keys, 1000), b)
    assert torch.equal(a, b)
    one = torch.empty(1, device=DEV, dtype=torch.int32)
    k().sample(logits[4:5], _rows(cfgs[4:5], keys[4:5], 1000), one)
    assert int(one[0]) == int(a[4])


def test_patch_tokens_takes_ids_that_are_still_on_the_device():
    ids = torch.tensor([11, 12, 13, 14, 15], dtype=torch.int32, device=DEV)
    src = torch.tensor([-1, 2, -1, 0, 0, 7, 7, 7], dtype=torch.int32, device=DEV)      # longer than ids: a graph's buffer
    prev = torch.tensor([100, 101, 102], dtype=torch.int32, device=DEV)
    k().patch_tokens(ids, src, prev)
    assert ids.tolist() == [11, 102, 13, 100, 100]


def test_stamps_follow_stream_order():
    slots = torch.zeros(4, dtype=torch.int64, device=DEV)
    x = torch.randn(1 << 20, device=DEV)
    k().stamp(slots, 0)
    for _ in range(4):
        x = x * 1.0001
    k().stamp(slots, 1)
    k().stamp(slots, 3)
    torch.cuda.synchronize()
    t = slots.tolist()
    assert 0 < t[0] <= t[1] <= t[3] and t[2] == 0


def test_device_error_words_are_clear_after_everything_above():
    k().check_device_errors()

