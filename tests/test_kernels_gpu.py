"""Numerics of every CUDA kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

from multimesh_jax_b200.ops import kernels as K

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device=DEV, dtype=torch.float32) * scale).to(dtype)


def _close(out, ref, rtol=2e-2, atol=None, frob=None):
    """Element-wise closeness plus a bound on the relative Frobenius error of the whole result:
    1e-2 for bf16 outputs (one rounding per element is 2^-9), 1e-3 for fp32 outputs. The
    element-wise bound alone scales with the largest reference value and would let a wrong
    low-magnitude column through."""
    ref = ref.float()
    if atol is None:
        atol = 2e-2 * max(ref.abs().max().item(), 1e-6)
    torch.testing.assert_close(out.float(), ref, rtol=rtol, atol=atol)
    if frob is None:
        frob = 1e-3 if out.dtype == torch.float32 else 1e-2
    err = ((out.float() - ref).norm() / ref.norm().clamp_min(1e-30)).item()
    assert err <= frob, f"relative Frobenius error {err:.3e} exceeds {frob:.1e}"


GEMM_SHAPES = [(128, 256, 64), (256, 512, 128), (384, 768, 320), (200, 264, 72), (1024, 1024, 1024),
               (4096, 5504, 4096), (104, 8, 8)]


@pytest.mark.parametrize("M,N,K_", GEMM_SHAPES)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_layouts(M, N, K_, a_mn, b_mn):
    torch.manual_seed(0)
    a = _rand(K_, M) if a_mn else _rand(M, K_)
    b = _rand(K_, N) if b_mn else _rand(N, K_)
    out = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    ref = (a.t() if a_mn else a).float() @ (b if b_mn else b.t()).float()
    assert K.read_status() == 0
    _close(out, ref)


@pytest.mark.parametrize("M,N,K_", GEMM_SHAPES)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_pair_layouts(M, N, K_, a_mn, b_mn):
    """CTA-pair kernel (cta_group::2, 256x256 tile per pair) against the fp32 product, ragged
    shapes included: rows of the second CTA of a pair may lie entirely outside the matrix."""
    torch.manual_seed(0)
    a = _rand(K_, M) if a_mn else _rand(M, K_)
    b = _rand(K_, N) if b_mn else _rand(N, K_)
    out = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, pair=True)
    ref = (a.t() if a_mn else a).float() @ (b if b_mn else b.t()).float()
    assert K.read_status() == 0
    _close(out, ref)


@pytest.mark.parametrize("count", [0, 1, 100, 256, 300, 1000, 1024, 5000])
def test_gemm_with_row_and_contraction_extents_read_on_the_device(count):
    """The GEMMs of a mixture-of-experts expert run over a receive region of fixed capacity and
    read how many of its rows hold tokens from device memory: forward / input-gradient form
    (the count limits M; rows of the output beyond it are left alone) and weight-gradient form
    (the count limits the contraction; the operands' rows up to the next multiple of 64 are
    zeroed first; a count of zero leaves the output untouched)."""
    torch.manual_seed(count)
    cap, D, F = 1024, 256, 384
    x = _rand(cap, D)
    w = _rand(F, D, scale=0.1)
    n = torch.tensor([count], dtype=torch.int32, device=DEV)
    live = min(count, cap)
    # forward form: y[:live] = x[:live] w^T, the rest keeps its sentinel
    y = torch.full((cap, F), 7.0, dtype=torch.bfloat16, device=DEV)
    K.linear_fwd(x, w, out=y, rows=n)
    if live:
        _close(y[:live], x[:live].float() @ w.float().t())
    assert bool((y[live:] == 7.0).all())
    # input-gradient form
    dy = _rand(cap, F)
    dx = torch.full((cap, D), 7.0, dtype=torch.bfloat16, device=DEV)
    K.linear_dgrad(dy, w, out=dx, rows=n)
    if live:
        _close(dx[:live], dy[:live].float() @ w.float())
    assert bool((dx[live:] == 7.0).all())
    # weight-gradient form: rows behind the count hold NaN until their tails are zeroed
    dy2, x2 = dy.clone(), x.clone()
    dy2[live:] = float("nan")
    x2[live:] = float("nan")
    K.zero_row_tail(dy2, n)
    K.zero_row_tail(x2, n)
    dw = torch.full((F, D), 3.0, dtype=torch.float32, device=DEV)
    K.linear_wgrad(dy2, x2, out=dw, rows=n)
    if live:
        _close(dw, dy[:live].float().t() @ x[:live].float())
    else:
        assert bool((dw == 3.0).all())
    # the element-wise kernels between the expert GEMMs honour the same count
    gu = _rand(cap, 2 * F)
    h = K.swiglu_fwd(gu, rows=n)
    if live:
        _close(h[:live], K.swiglu_fwd(gu[:live].contiguous()))
    dh = _rand(cap, F)
    dgu = K.swiglu_bwd(gu, dh, rows=n)
    if live:
        _close(dgu[:live], K.swiglu_bwd(gu[:live].contiguous(), dh[:live].contiguous()))
    assert K.read_status() == 0


def test_gemm_pair_accumulates_into_fp32():
    torch.manual_seed(1)
    T, Kd, N = 2048, 512, 768
    x, dy = _rand(T, Kd), _rand(T, N)
    dw = torch.zeros(N, Kd, device=DEV, dtype=torch.float32)
    for _ in range(2):
        K.gemm(dy, x, a_mn=True, b_mn=True, out=dw, accumulate=True, pair=True)
    assert K.read_status() == 0
    _close(dw, 2 * dy.float().t() @ x.float(), rtol=1e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_accumulate(dtype):
    torch.manual_seed(1)
    M, N, K_ = 512, 768, 256
    a, b = _rand(M, K_), _rand(N, K_)
    c0 = torch.randn(M, N, device=DEV).to(dtype)
    c = c0.clone()
    K.gemm(a, b, out=c, accumulate=True)
    ref = c0.float() + a.float() @ b.float().t()
    assert K.read_status() == 0
    _close(c, ref)
    c2 = torch.empty(M, N, device=DEV, dtype=torch.float32)
    K.gemm(a, b, out=c2)
    _close(c2, a.float() @ b.float().t(), rtol=1e-3)


def test_gemm_strided_operands():
    torch.manual_seed(2)
    big = _rand(512, 3 * 256)
    x = big[:, 256:512]          # row stride 768, unit inner stride
    w = _rand(384, 256)
    out = K.linear_fwd(x, w)
    _close(out, x.float() @ w.float().t())
    outbuf = torch.zeros(512, 1024, device=DEV, dtype=torch.bfloat16)
    K.linear_fwd(x, w, out=outbuf[:, 128:512])
    _close(outbuf[:, 128:512], x.float() @ w.float().t())
    assert outbuf[:, :128].abs().max().item() == 0 and outbuf[:, 512:].abs().max().item() == 0


def test_linear_grads():
    torch.manual_seed(3)
    T, Kd, N = 1024, 512, 768
    x, w, dy = _rand(T, Kd), _rand(N, Kd, scale=0.05), _rand(T, N)
    _close(K.linear_dgrad(dy, w), dy.float() @ w.float())
    dw = torch.zeros(N, Kd, device=DEV, dtype=torch.float32)
    K.linear_wgrad(dy, x, out=dw, accumulate=True)
    K.linear_wgrad(dy, x, out=dw, accumulate=True)
    _close(dw, 2 * dy.float().t() @ x.float(), rtol=1e-3)
    assert K.read_status() == 0


@pytest.mark.parametrize("D", [512, 4096, 8192])
def test_rmsnorm(D):
    torch.manual_seed(4)
    rows = 333
    x, w, dy = _rand(rows, D), _rand(D, scale=0.5) + 1, _rand(rows, D)
    y, rstd = K.rmsnorm_fwd(x, w, 1e-5)
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    _close(y, ref.detach())
    ref.backward(dy.float())
    dx, dw = K.rmsnorm_bwd(x, w, dy, rstd)
    _close(dx, xf.grad)
    _close(dw, wf.grad, rtol=1e-2)
    base = _rand(rows, D)
    acc = base.clone()
    K.rmsnorm_bwd(x, w, dy, rstd, dx_inout=acc)
    _close(acc, base.float() + xf.grad)


def test_rope_roundtrip_and_reference():
    torch.manual_seed(5)
    B, S, H, Dh = 2, 128, 4, 128
    cos, sin = K.rope_tables(S, Dh, 1e4, DEV)
    qkv = _rand(B * S, 3 * H * Dh)
    q = qkv[:, : H * Dh].view(B * S, H, Dh)
    q0 = q.clone()
    ref = K.rope_(q0.cpu().clone(), cos.cpu(), sin.cpu())
    K.rope_(q, cos, sin)
    _close(q, ref.to(DEV))
    K.rope_(q, cos, sin, backward=True)
    _close(q, q0, rtol=3e-2, frob=1.5e-2)


def test_swiglu():
    torch.manual_seed(6)
    T, F = 257, 1376
    gu, dh = _rand(T, 2 * F), _rand(T, F)
    guf = gu.float().requires_grad_(True)
    ref = torch.nn.functional.silu(guf[:, :F]) * guf[:, F:]
    _close(K.swiglu_fwd(gu), ref.detach())
    ref.backward(dh.float())
    _close(K.swiglu_bwd(gu, dh), guf.grad)


@pytest.mark.parametrize("V", [32000, 1000, 1003])
def test_cross_entropy(V):
    torch.manual_seed(7)
    rows = 64
    ld = (V + 7) // 8 * 8
    buf = _rand(rows, ld, scale=2.0)
    logits = buf[:, :V]
    tgt = torch.randint(0, V, (rows,), device=DEV)
    tgt[3] = -100
    lf = logits.float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lf, tgt, ignore_index=-100, reduction="none")
    (ref.sum() * 0.5).backward()
    loss = K.cross_entropy_fwd_bwd(logits, tgt, 0.5)
    _close(loss, ref.detach(), rtol=1e-3, atol=1e-3)
    _close(logits, lf.grad, atol=2e-3)


def test_embedding():
    torch.manual_seed(8)
    V, D, T = 1000, 256, 777
    table = _rand(V, D)
    ids = torch.randint(0, V, (T,), device=DEV)
    out = K.embedding_fwd(table, ids)
    assert torch.equal(out, table[ids])
    dout = _rand(T, D)
    grad = torch.zeros(V, D, device=DEV)
    K.embedding_bwd(dout, ids, grad)
    ref = torch.zeros(V, D, device=DEV).index_add_(0, ids, dout.float())
    _close(grad, ref, rtol=1e-3)


def test_adamw_matches_torch():
    torch.manual_seed(9)
    n = 4096 * 3
    p = torch.randn(n, device=DEV)
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    master, m, v = p.clone(), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    work = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    for step in range(1, 4):
        g = torch.randn(n, device=DEV)
        ref_p.grad = g.clone()
        opt.step()
        K.adamw_step_(master, work, m, v, g, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8,
                      weight_decay=0.1, step=step)
    torch.testing.assert_close(master, ref_p.data, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(work.float(), master, rtol=1e-2, atol=1e-2)


def test_add_and_accumulate():
    a, b = _rand(1000, 64), _rand(1000, 64)
    _close(K.add(a, b), a.float() + b.float())
    acc = torch.randn(1000, 64, device=DEV)
    ref = acc + b.float()
    K.accumulate_(acc, b)
    torch.testing.assert_close(acc, ref)
    s = torch.zeros(1, device=DEV)
    K.sumsq(acc, s)
    torch.testing.assert_close(s[0], (acc.double() ** 2).sum().float(), rtol=1e-4, atol=1e-3)


def test_bounded_flag_wait_expires_with_a_status_and_the_context_stays_usable():
    """A wait on a flag that nothing raises gives up after its time limit, records the expiry in
    the device status word and lets the stream continue; later kernels run normally."""
    from multimesh_jax_b200.parallel import symm
    dev = torch.device("cuda", 0)
    K.read_status()                       # clear
    arena = symm.SymmetricArena(1 << 20, dev)
    off = arena.alloc_flag()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    symm.wait_flags(arena, [arena.flag_ptr(arena.rank, off)], 1, limit_ms=300)
    t1.record()
    torch.cuda.synchronize()
    assert 250 <= t0.elapsed_time(t1) < 5000
    assert K.read_status() == 5           # MM_ERR_WAIT_PEER; reading clears it
    # a raised flag lets the same wait pass at once, and ordinary work still runs
    symm.set_flags(arena, [arena.flag_ptr(arena.rank, off)], 1)
    symm.wait_flags(arena, [arena.flag_ptr(arena.rank, off)], 1, limit_ms=300)
    x = torch.randn(256, 512, device=dev).bfloat16()
    y = K.linear_fwd(x, x)
    torch.cuda.synchronize()
    assert K.read_status() == 0 and torch.isfinite(y.float()).all()
    arena.close()


def test_moe_router_dispatch_is_total_for_nan_and_infinite_logits():
    """Tokens whose router logits are all NaN or -inf still pick valid, distinct experts (the
    kernel's rule is restated by ``moe.select_experts``), every row lands inside its expert's
    receive region and the status word stays clear."""
    from multimesh_jax_b200.ops import moe
    from multimesh_jax_b200.parallel import symm
    from multimesh_jax_b200.parallel.ep import PeerMoE
    torch.manual_seed(5)
    T, D, E, k = 64, 256, 4, 2
    x = _rand(T, D)
    wr = _rand(E, D, scale=0.5)
    x[3] = float("nan")                    # NaN logits for token 3
    x[7] = 0.0                             # all logits equal: ties go to the lowest index
    wr_inf = wr.clone()
    arena = symm.SymmetricArena(16 << 20, torch.device("cuda", 0))
    pm = PeerMoE(arena, [arena.rank], T, D, E)
    pm.k = k
    for weights in (wr, wr_inf):
        idx, gates, slot = pm._route_dispatch(x, weights, None)
        torch.cuda.synchronize()
        assert K.read_status() == 0
        logits = x.float() @ weights.float().t()
        want, _ = moe.select_experts(logits.cpu(), k)
        # ordinary tokens can differ from the fp32 product only on near-ties; the degenerate ones must match
        assert idx[3].tolist() == want[3].tolist() == [0, 1]
        assert idx[7].tolist() == want[7].tolist() == [0, 1]
        assert int(idx.min()) >= 0 and int(idx.max()) < E
        assert bool((idx[:, 0] != idx[:, 1]).all())
        assert int(slot.min()) >= 0 and int(slot.max()) < pm.capacity
        agree = (idx.cpu().long() == want).all(dim=1).float().mean().item()
        assert agree > 0.95, agree
        counts = pm._counts()
        assert sum(counts) == T * k
    arena.close()
