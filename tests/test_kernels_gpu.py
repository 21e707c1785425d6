"""Numerics of every CUDA kernel against a plain PyTorch fp32 definition of the same op (B200 only)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()


@pytest.fixture(scope="module")
def dev(bmt_gpu):
    return torch.device("cuda")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(128, 128, 64), (1024, 2560, 2560), (1000, 2568, 520), (333, 80, 96), (2048, 8192, 2560)])
def test_gemm_layouts(dev, dtype, shape):
    from bmtrain_b200.ops import gemm as G

    m, n, k = shape
    torch.manual_seed(1)
    tol = 6e-3 if dtype == torch.bfloat16 else 1e-3
    a = torch.randn(m, k, device=dev, dtype=dtype)
    b = torch.randn(n, k, device=dev, dtype=dtype)
    bias = torch.randn(n, device=dev, dtype=dtype)
    ref = a.float() @ b.float().t()
    assert _rel(G.gemm_nt(a, b), ref) < tol
    assert _rel(G.gemm_nt(a, b, bias, "relu"), torch.relu(ref + bias.float())) < tol
    assert _rel(G.gemm_nt(a, b, bias, "gelu"), torch.nn.functional.gelu(ref + bias.float())) < tol
    bk = torch.randn(k, n, device=dev, dtype=dtype)
    assert _rel(G.gemm_nn(a, bk), a.float() @ bk.float()) < tol
    at = torch.randn(k, m, device=dev, dtype=dtype)
    assert _rel(G.gemm_tn(at, bk), at.float().t() @ bk.float()) < tol
    acc = torch.randn(m, n, device=dev, dtype=torch.float32)
    expect = acc + at.float().t() @ bk.float()
    G.gemm_tn(at, bk, out=acc, accumulate=True)
    assert _rel(acc, expect) < 1e-4
    from bmtrain_b200.ops import _native
    assert _native.cuda_lib().bmt_gemm_status() == 0


def test_linear_autograd(dev):
    from bmtrain_b200.ops import gemm as G

    torch.manual_seed(2)
    x = torch.randn(4, 96, 256, device=dev, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(512, 256, device=dev) * 0.05).to(torch.bfloat16).requires_grad_()
    b = torch.randn(512, device=dev, dtype=torch.bfloat16, requires_grad=True)
    y = G.linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = x.detach().float().requires_grad_(), w.detach().float().requires_grad_(), b.detach().float().requires_grad_()
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    assert _rel(y, yr) < 6e-3 and _rel(x.grad, xr.grad) < 6e-3 and _rel(w.grad, wr.grad) < 6e-3 and _rel(b.grad, br.grad) < 6e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_adam_multi(dev, dtype):
    from bmtrain_b200.ops import adam as A

    torch.manual_seed(3)
    entries, refs = [], []
    for n in (8, 1000, 4099, 1 << 20):
        p32 = torch.randn(n, device=dev)
        g = (torch.randn(n, device=dev) * 64).to(dtype)
        m = (torch.randn(n, device=dev) * 0.1).to(torch.float16 if dtype == torch.float16 else torch.float32)
        v = torch.rand(n, device=dev) * 0.1
        p16 = p32.to(dtype)
        entries.append((p32, p16, g, m, v))
        refs.append(tuple(t.cpu().clone() for t in (p32, p16, g, m, v)))
    A.adam_half_multi(entries, 0.9, 0.999, 1e-8, 1e-3, 64.0, 0.01, 7)
    A.adam_half_multi(refs, 0.9, 0.999, 1e-8, 1e-3, 64.0, 0.01, 7)  # CPU tensors: PyTorch definition
    for e, r in zip(entries, refs):
        assert torch.allclose(e[0].cpu(), r[0], atol=1e-5, rtol=1e-5)
        assert torch.allclose(e[1].cpu().float(), r[1].float(), atol=1e-2, rtol=1e-2)
        assert torch.allclose(e[3].cpu().float(), r[3].float(), atol=2e-3, rtol=2e-3)
        assert torch.allclose(e[4].cpu(), r[4], atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_has_inf_nan(dev, dtype):
    from bmtrain_b200.ops.infnan import has_inf_nan

    torch.manual_seed(4)
    for n in (1, 7, 31, 1000, 4097, 100000, 1000003):
        x = torch.randn(n, device=dev, dtype=dtype)
        flag = torch.zeros(1, dtype=torch.uint8, device=dev)
        has_inf_nan(x, flag)
        assert flag.item() == 0
        for bad in (float("inf"), float("-inf"), float("nan")):
            y = x.clone()
            y[torch.randint(0, n, (1,)).item()] = bad
            flag.zero_()
            has_inf_nan(y, flag)
            assert flag.item() == 1, (n, bad)
    # a misaligned slice is scanned correctly
    base = torch.zeros(1001, device=dev, dtype=dtype)
    base[0] = float("nan")
    flag = torch.zeros(1, dtype=torch.uint8, device=dev)
    has_inf_nan(base[1:], flag)
    assert flag.item() == 0


def test_sq_norm_and_scale(dev):
    from bmtrain_b200.ops import infnan

    torch.manual_seed(5)
    ts = [torch.randn(n, device=dev, dtype=torch.bfloat16) for n in (5, 1000, 70001)]
    out = torch.zeros(1, device=dev)
    infnan.multi_sq_norm(ts, out)
    ref = sum(t.float().pow(2).sum() for t in ts)
    assert abs(out.item() - ref.item()) / ref.item() < 1e-4
    before = [t.clone() for t in ts]
    infnan.multi_scale(ts, torch.tensor([0.5], device=dev))
    for t, b in zip(ts, before):
        assert torch.allclose(t.float(), b.float() * 0.5, atol=1e-2, rtol=1e-2)
    infnan.multi_scale(ts, torch.tensor([3.0], device=dev))  # coefficients >= 1 leave the data alone
    for t, b in zip(ts, before):
        assert torch.allclose(t.float(), b.float() * 0.5, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("classes", [10, 1000, 10240, 30000, 32003])
def test_cross_entropy(dev, dtype, classes):
    import bmtrain_b200 as bmt

    torch.manual_seed(6)
    n = 77
    x = torch.randn(n, classes, device=dev, dtype=dtype, requires_grad=True)
    t = torch.randint(0, classes, (n,), device=dev)
    t[::7] = -100
    w = torch.rand(classes, device=dev)
    for weight in (None, w):
        loss = bmt.loss.FusedCrossEntropy(weight=weight)(x, t)
        (loss * 32768).backward()
        xr = x.detach().float().requires_grad_()
        ref = torch.nn.functional.cross_entropy(xr, t, weight=weight)
        (ref * 32768).backward()
        assert abs(loss.item() - ref.item()) < 1e-3 if dtype == torch.bfloat16 else abs(loss.item() - ref.item()) < 1e-4
        assert (x.grad.float() - xr.grad).abs().max().item() < (4.0 if dtype == torch.bfloat16 else 0.5)
        x.grad = None


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rms", [False, True])
def test_norms(dev, dtype, rms):
    from bmtrain_b200.ops import norm as N

    torch.manual_seed(7)
    for rows, d in ((5, 64), (300, 2560), (64, 8192)):
        x = torch.randn(rows, d, device=dev, dtype=dtype, requires_grad=True)
        w = (1 + 0.1 * torch.randn(d, device=dev)).to(dtype).requires_grad_()
        b = (0.1 * torch.randn(d, device=dev)).to(dtype).requires_grad_()
        g = torch.randn(rows, d, device=dev, dtype=dtype)
        y = N.rms_norm(x, w, 1e-5) if rms else N.layer_norm(x, w, b, 1e-5)
        y.backward(g)
        xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
        if rms:
            yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
        else:
            yr = torch.nn.functional.layer_norm(xr, (d,), wr, br, 1e-5)
        yr.backward(g.float())
        tol = 2e-2 if dtype == torch.bfloat16 else 3e-3
        assert _rel(y, yr) < tol and _rel(x.grad, xr.grad) < tol and _rel(w.grad, wr.grad) < tol
        if not rms:
            assert _rel(b.grad, br.grad) < tol


def test_embedding(dev):
    from bmtrain_b200.ops import embedding as E

    torch.manual_seed(8)
    w = torch.randn(1000, 256, device=dev, dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, 1000, (4, 33), device=dev)
    out = E.embedding(ids, w)
    assert torch.equal(out, w[ids])
    g = torch.randn_like(out)
    out.backward(g)
    ref = torch.zeros(1000, 256, device=dev)
    ref.index_add_(0, ids.reshape(-1), g.reshape(-1, 256).float())
    assert _rel(w.grad, ref) < 1e-2
    neg = ids.clone()
    neg[0, :5] = -1
    out2 = E.embedding_forward(neg, w.detach())
    assert out2[0, :5].abs().max().item() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("cfg", [(2, 128, 4, 4, 64, False, True), (2, 512, 8, 8, 80, False, True),
                                 (1, 256, 8, 2, 128, True, False), (3, 100, 2, 2, 64, True, False)])
def test_attention(dev, dtype, cfg):
    from bmtrain_b200.ops import attention as AT

    b, s, h, hk, d, causal, dense = cfg
    torch.manual_seed(9)
    q = torch.randn(b, s, h, d, device=dev, dtype=dtype, requires_grad=True)
    k = torch.randn(b, s, hk, d, device=dev, dtype=dtype, requires_grad=True)
    v = torch.randn(b, s, hk, d, device=dev, dtype=dtype, requires_grad=True)
    mask = None
    if dense:
        valid = torch.arange(s, device=dev)[None] < torch.tensor([s - 3 * i for i in range(b)], device=dev)[:, None]
        mask = valid[:, None, :] & valid[:, :, None] & torch.ones(s, s, dtype=torch.bool, device=dev).tril()[None]
    out = AT.attention(q, k, v, causal=causal, mask=mask)
    g = torch.randn_like(out)
    out.backward(g)
    qr, kr, vr = (t.detach().float().cpu().requires_grad_() for t in (q, k, v))
    ref = AT._reference_attention(qr, kr, vr, 1.0 / math.sqrt(d), causal, None if mask is None else mask.cpu(), None)
    ref.backward(g.float().cpu())
    tol = 3e-2 if dtype == torch.bfloat16 else 5e-3
    assert _rel(out.cpu(), ref) < tol
    assert _rel(q.grad.cpu(), qr.grad) < tol and _rel(k.grad.cpu(), kr.grad) < tol and _rel(v.grad.cpu(), vr.grad) < tol


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("cfg", [
    # b, sq, sk, h, hk, d, causal, masking
    (2, 128, 128, 4, 4, 64, True, None), (2, 512, 512, 8, 8, 80, True, None), (1, 300, 300, 8, 2, 128, True, None),
    (2, 256, 384, 4, 2, 64, True, "lens"), (2, 200, 200, 4, 4, 96, False, "dense"), (3, 100, 260, 2, 1, 32, False, "lens"),
    (1, 1024, 1024, 4, 4, 128, True, None), (1, 130, 130, 2, 2, 16, False, None)])
def test_flash_attention_forward(dev, dtype, cfg):
    """Fused tcgen05 attention forward against the fp32 definition: output and log-sum-exp, strided (packed QKV) inputs,
    grouped-query heads, causal / key-length / dense masks, ragged tile edges and rows with no visible key."""
    from bmtrain_b200.ops import attention as AT
    from bmtrain_b200.ops import _native

    b, sq, sk, h, hk, d, causal, masking = cfg
    torch.manual_seed(13)
    g = h // hk
    # q, k, v as strided views of one packed projection, the way the models produce them
    packed_q = torch.randn(b, sq, hk, g + 2, d, device=dev, dtype=dtype)
    packed_kv = packed_q if sk == sq else torch.randn(b, sk, hk, g + 2, d, device=dev, dtype=dtype)
    q = packed_q[:, :, :, :g].reshape(b, sq, h, d)
    k, v = packed_kv[:, :, :, g], packed_kv[:, :, :, g + 1]
    mask = lens = None
    if masking == "lens":
        lens = torch.tensor([max(1, sk - 37 * i) for i in range(b)], device=dev, dtype=torch.int32)
        if b > 2:
            lens[-1] = 0     # a sample without any visible key: zeros out, -inf log-sum-exp
    if masking == "dense":
        mask = torch.rand(b, sq, sk, device=dev) > 0.3
        mask[:, 5] = False   # a fully masked row
    assert AT.flash_usable(q, k, v)
    m8, l32 = AT._softmax_args(mask, lens)
    scale = 1.0 / math.sqrt(d)
    out, lse = AT.flash_forward(q, k, v, scale, causal, m8, l32)
    torch.cuda.synchronize()
    assert _native.cuda_lib().bmt_attn_status() == 0
    ref = AT._reference_attention(q.float().cpu(), k.float().cpu(), v.float().cpu(), scale, causal,
                                  None if mask is None else mask.cpu(), None if lens is None else lens.cpu())
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    assert torch.isfinite(out).all()
    assert _rel(out.float().cpu(), ref.float()) < tol
    # log-sum-exp against the definition
    kk = k.float().cpu().repeat_interleave(g, dim=2)
    sc = torch.einsum("bqhd,bkhd->bhqk", q.float().cpu(), kk) * scale
    keep = torch.ones(b, 1, sq, sk, dtype=torch.bool)
    if causal:
        keep = keep & torch.ones(sq, sk, dtype=torch.bool).tril(sk - sq)
    if mask is not None:
        keep = keep & mask.cpu().view(b, 1, sq, sk)
    if lens is not None:
        keep = keep & (torch.arange(sk)[None, None, None, :] < lens.cpu().view(b, 1, 1, 1))
    want = torch.logsumexp(sc.masked_fill(~keep, float("-inf")), dim=-1)
    got = lse.cpu()
    finite = torch.isfinite(want)
    assert torch.equal(torch.isfinite(got), finite)
    assert (got[finite] - want[finite]).abs().max().item() < (5e-2 if dtype == torch.bfloat16 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("cfg", [
    (2, 128, 128, 4, 4, 64, True, None), (2, 512, 512, 8, 8, 80, True, None), (1, 300, 300, 8, 2, 128, True, None),
    (2, 256, 384, 4, 2, 64, True, "lens"), (2, 200, 200, 4, 4, 96, False, "dense"), (3, 100, 260, 2, 1, 32, False, "lens"),
    (1, 640, 640, 2, 2, 128, True, "dense")])
def test_flash_attention_backward(dev, dtype, cfg):
    """Fused attention backward (dq, dk, dv) through autograd against the fp32 definition."""
    from bmtrain_b200.ops import attention as AT
    from bmtrain_b200.ops import _native

    b, sq, sk, h, hk, d, causal, masking = cfg
    torch.manual_seed(14)
    q = torch.randn(b, sq, h, d, device=dev, dtype=dtype, requires_grad=True)
    k = torch.randn(b, sk, hk, d, device=dev, dtype=dtype, requires_grad=True)
    v = torch.randn(b, sk, hk, d, device=dev, dtype=dtype, requires_grad=True)
    mask = lens = None
    if masking == "lens":
        lens = torch.tensor([max(1, sk - 37 * i) for i in range(b)], device=dev, dtype=torch.int32)
        if b > 2:
            lens[-1] = 0
    if masking == "dense":
        mask = torch.rand(b, sq, sk, device=dev) > 0.3
        if causal:
            mask = mask & torch.ones(sq, sk, dtype=torch.bool, device=dev).tril(sk - sq)
        mask[:, 5] = False
    assert AT.flash_usable(q, k, v)
    out = AT.attention(q, k, v, causal=causal, mask=mask, kv_lens=lens)
    g = torch.randn_like(out)
    out.backward(g)
    torch.cuda.synchronize()
    assert _native.cuda_lib().bmt_attn_status() == 0
    qr, kr, vr = (t.detach().float().cpu().requires_grad_() for t in (q, k, v))
    ref = AT._reference_attention(qr, kr, vr, 1.0 / math.sqrt(d), causal, None if mask is None else mask.cpu(),
                                  None if lens is None else lens.cpu())
    ref.backward(g.float().cpu())
    tol = 3e-2 if dtype == torch.bfloat16 else 6e-3
    assert _rel(out.float().cpu(), ref) < tol
    for name, got, want in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        assert torch.isfinite(got).all(), name
        assert _rel(got.float().cpu(), want) < tol, name


def test_swiglu_colsum(dev):
    from bmtrain_b200.ops import elementwise as EW, gemm as G

    torch.manual_seed(10)
    x = torch.randn(100, 2 * 512, device=dev, dtype=torch.bfloat16, requires_grad=True)
    y = EW.swiglu(x)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = torch.nn.functional.silu(xr[:, :512]) * xr[:, 512:]
    yr.backward(g.float())
    assert _rel(y, yr) < 2e-2 and _rel(x.grad, xr.grad) < 2e-2
    z = torch.randn(1000, 520, device=dev, dtype=torch.float16)
    assert _rel(G.bias_grad(z), z.float().sum(0)) < 2e-3
    # many rows: the grid is split over the rows, the last CTA of a column block adds the partial sums; the second call
    # finds the ticket counters where the first one left them
    for _ in range(2):
        z = torch.randn(8192 + 77, 2560, device=dev, dtype=torch.bfloat16)
        assert _rel(G.bias_grad(z), z.float().sum(0)) < 4e-3


@pytest.mark.parametrize("dtype,act", [(torch.float16, "gelu"), (torch.bfloat16, "gelu"), (torch.float16, "relu")])
def test_fused_gpt_block_matches_oracle(dev, dtype, act):
    """The native block executor against the plain PyTorch fp32 block (forward, input gradient, every parameter gradient).

    With ReLU a handful of pre-activations that sit within half-precision rounding of zero get the other side of the
    kink than in the fp32 oracle, which moves single gradient entries by a whole term; gradients are therefore held
    to a loose bound there and to the tight one with the smooth GELU."""
    import bmtrain_b200 as bmt
    from oracle import OracleBlock

    torch.manual_seed(11)
    d, dh, h, dff, b, s = 256, 64, 4, 1024, 2, 100
    blk = bmt.models.TransformerEncoder(d, dh, h, dff, bias=True, dtype=dtype, activation=act)
    ref = OracleBlock(d, dh, h, dff, True, act)
    with torch.no_grad():
        for p in ref.parameters():
            p.normal_(0, 0.05)
        ref.ln_attn.weight.add_(1.0)
        ref.ln_ff.weight.add_(1.0)
    blk.load_state_dict(ref.state_dict())
    x = torch.randn(b, s, d, device=dev, dtype=dtype, requires_grad=True)
    valid = torch.arange(s, device=dev)[None] < torch.tensor([s, s - 9], device=dev)[:, None]
    mask = valid[:, None, :] & valid[:, :, None] & torch.ones(s, s, dtype=torch.bool, device=dev).tril()[None]
    y = blk(x, mask)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().cpu().requires_grad_()
    yr = ref(xr, mask.cpu())
    yr.backward(g.float().cpu())
    tol = 4e-2 if dtype == torch.bfloat16 else 6e-3
    assert _rel(y.cpu(), yr) < tol
    gtol = 0.25 if act == "relu" else 4e-2 if dtype == torch.bfloat16 else 2e-2
    assert _rel(x.grad.cpu(), xr.grad) < gtol
    mine = dict(blk.named_parameters())
    for name, p in ref.named_parameters():
        got = mine[name].grad
        assert got is not None, name
        assert _rel(got.cpu().view(p.shape), p.grad) < gtol, name


def test_fused_gpt_block_accumulates_into_attached_gradients(dev):
    """When every parameter already has a gradient buffer (as inside a ZeRO block), the executor adds weight, bias and norm
    gradients in place: a second identical backward pass doubles them, and no gradient tensor goes back to autograd."""
    import bmtrain_b200 as bmt

    torch.manual_seed(13)
    d, dh, h, dff, b, s = 256, 64, 4, 1024, 2, 128
    blk = bmt.models.TransformerEncoder(d, dh, h, dff, bias=True, dtype=torch.bfloat16, activation="gelu")
    with torch.no_grad():
        for p in blk.parameters():
            p.normal_(0, 0.05)
    x = torch.randn(b, s, d, device=dev, dtype=torch.bfloat16)
    mask = torch.ones(s, s, dtype=torch.bool, device=dev).tril()[None].expand(b, -1, -1).contiguous()
    g = torch.randn(b, s, d, device=dev, dtype=torch.bfloat16)
    blk(x, mask).backward(g)
    first = {n: p.grad.clone() for n, p in blk.named_parameters()}
    ptrs = {n: p.grad.data_ptr() for n, p in blk.named_parameters()}
    blk(x, mask).backward(g)
    torch.cuda.synchronize()
    for n, p in blk.named_parameters():
        assert p.grad.data_ptr() == ptrs[n], n
        assert _rel(p.grad, 2 * first[n].float()) < 1e-2, n


@pytest.mark.parametrize("math", ["gpu", "auto"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_offload_adam_gpu_streamed_matches_host_math(dev, dtype, math):
    """AdamOffloadOptimizer: the GPU-streamed step (state chunks host -> HBM -> host) and the host AVX step give the same
    parameters and the same host-resident state; both follow an fp32 AdamW run."""
    import bmtrain_b200 as bmt

    torch.manual_seed(12)
    shapes = [(1 << 24) + 4096, 2560, (3000, 512), (1 << 23)]
    w0 = [torch.randn(s, device=dev) * 0.1 for s in shapes]
    ref = [w.clone().requires_grad_() for w in w0]
    o_ref = torch.optim.AdamW(ref, lr=1e-2, weight_decay=1e-2)
    pa = [torch.nn.Parameter(w.to(dtype)) for w in w0]
    pb = [torch.nn.Parameter(w.to(dtype)) for w in w0]
    oa = bmt.optim.AdamOffloadOptimizer(pa, lr=1e-2, weight_decay=1e-2, math=math)
    ob = bmt.optim.AdamOffloadOptimizer(pb, lr=1e-2, weight_decay=1e-2, math="cpu")
    scale = 64.0
    for step in range(4):
        for r, a, b in zip(ref, pa, pb):
            g = torch.randn_like(r)
            r.grad = g.clone()
            a.grad = (g * scale).to(dtype)
            b.grad = (g * scale).to(dtype)
        o_ref.step(); oa.step(scale=scale); ob.step(scale=scale)
    torch.cuda.synchronize()
    sa, sb = oa.state_dict(), ob.state_dict()
    tol = 3e-2 if dtype == torch.bfloat16 else 4e-3
    for i, (r, a, b) in enumerate(zip(ref, pa, pb)):
        assert (a.float() - b.float()).abs().max().item() <= (1e-2 if dtype == torch.bfloat16 else 2e-3)
        assert (a.float() - r).abs().max().item() < tol
        for key in ("exp_avg", "exp_avg_sq", "_param_fp32"):
            assert not sa["state"][i][key].is_cuda
            assert torch.allclose(sa["state"][i][key], sb["state"][i][key], atol=1e-5, rtol=1e-4), (i, key)


def test_peer_copy_and_fused_helpers(dev):
    """Small native helpers of the peer-memory runtime that need no second GPU: the SM copy kernel (here local to local),
    the pusher-count heuristic and the fused kernels' timing counters."""
    import ctypes

    from bmtrain_b200.ops import _native
    from bmtrain_b200.parallel import fused_ops

    lib = _native.cuda_lib()
    src = torch.randint(0, 255, (3 * 1024 * 1024 + 48,), dtype=torch.uint8, device=dev)
    dst = torch.zeros_like(src)
    for grid in (1, 37, 148):
        dst.zero_()
        _native.check(lib.bmt_peer_copy(_native.ptr(dst), _native.ptr(src), ctypes.c_int64(src.numel()), ctypes.c_int(grid),
                                        _native.stream_handle()), "peer copy")
        assert torch.equal(dst, src)
    assert lib.bmt_peer_copy(_native.ptr(dst), _native.ptr(src), ctypes.c_int64(17), ctypes.c_int(4), _native.stream_handle()) != 0
    # compute-bound problems get few pusher CTAs, transfer-bound ones many; always a multiple of 4 that leaves SMs for math
    few = lib.bmt_fused_comm_ctas(ctypes.c_double(6.4e11), ctypes.c_double(4e7), ctypes.c_double(4e7))
    many = lib.bmt_fused_comm_ctas(ctypes.c_double(4e10), ctypes.c_double(4e7), ctypes.c_double(4e7))
    assert 8 <= few < many <= 116 and few % 4 == 0 and many % 4 == 0
    stats = fused_ops.kernel_stats()
    assert stats["kernels"] == 0 and stats["pusher_us_max"] == 0.0


def test_bounded_wait_reports_instead_of_hanging(dev):
    """A kernel that waits for a flag nobody sets gives up after its time limit, records a status code and leaves the
    context usable (the host-visible form of a peer that never arrives)."""
    import ctypes
    import time

    from bmtrain_b200.ops import _native

    lib = _native.cuda_lib()
    world = 2
    flags = torch.zeros(8 * world, dtype=torch.int32, device=dev)           # one flag row per slot, never written
    table = torch.tensor([flags.data_ptr()] * world, dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    t0 = time.perf_counter()
    _native.check(lib.bmt_symm_signal_wait(ctypes.c_void_p(table.data_ptr()), ctypes.c_int(world), ctypes.c_int(0), ctypes.c_int(3),
                                           ctypes.c_uint(1), ctypes.c_int(0), ctypes.c_int(1), _native.ptr(status),
                                           ctypes.c_double(0.2), _native.stream_handle()), "signal/wait kernel")
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 0.15 < waited < 5.0, waited
    assert int(status.item()) == (0x200 | 0)
    # a wait whose flag is there returns at once and does not touch the status word
    flags[3 * world:4 * world] = 1
    status.zero_()
    _native.check(lib.bmt_symm_signal_wait(ctypes.c_void_p(table.data_ptr()), ctypes.c_int(world), ctypes.c_int(0), ctypes.c_int(3),
                                           ctypes.c_uint(1), ctypes.c_int(0), ctypes.c_int(1), _native.ptr(status),
                                           ctypes.c_double(0.2), _native.stream_handle()), "signal/wait kernel")
    assert int(status.item()) == 0
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0  # the context still works
